"""CPU tests of the buffer arithmetic behind deepwell_b200.exchange.QuantizedRowExchange: which bytes of a slot hold which
rows, for every rank count the bench runs.  The exchange itself (peer copies over NVLink) is checked byte for byte
inside `bench.py --gpus N` (key `exchange.parity`)."""
import numpy as np
import pytest

from deepwell_b200.exchange import SlotLayout
from oracle import mx_oracle as o


@pytest.mark.parametrize("world", [2, 4, 8])
def test_slices_and_local_rows_tile_each_buffer_exactly_once(world):
    shapes = [(128 * world * 2, 96), (128 * world, 4096 + 32), (128 * world * 3, 32)]
    lay = SlotLayout(shapes, world)
    end = 0
    for (rows, cols), (c_off, c_bytes, s_off, s_bytes) in zip(shapes, lay.offsets):
        assert c_off % 256 == 0 and s_off % 256 == 0 and c_off >= end and s_off >= c_off + c_bytes
        assert c_bytes == rows * cols and s_bytes == o.sf_tiled_size(rows, cols // 32)
        end = s_off + s_bytes
    assert lay.slot_bytes >= end
    for i, (rows, cols) in enumerate(shapes):
        for shared in (rows, rows - 128 * world, 128 * world, 0):
            seen_c = np.zeros(lay.offsets[i][1], dtype=np.int32)
            seen_s = np.zeros(lay.offsets[i][3], dtype=np.int32)
            pieces = [lay.rows_of(shared, r) for r in range(world)] + [(shared, rows)]      # the ranks' slices + the local rows
            assert all(r0 % 128 == 0 and r1 % 128 == 0 for r0, r1 in pieces)
            for r0, r1 in pieces:
                c_lo, c_hi, s_lo, s_hi = lay.byte_ranges(i, r0, r1)
                seen_c[c_lo:c_hi] += 1
                seen_s[s_lo:s_hi] += 1
            assert (seen_c == 1).all() and (seen_s == 1).all()


def test_shared_rows_are_validated():
    lay = SlotLayout([(1024, 64), (2048, 64)], 4)
    assert lay.check_shared_rows(None) == [1024, 2048]
    assert lay.check_shared_rows([512, 0]) == [512, 0]
    for bad in ([512], [100, 0], [1536, 0], [-512, 0]):
        with pytest.raises(ValueError):
            lay.check_shared_rows(bad)
    with pytest.raises(ValueError):
        SlotLayout([(1000, 64)], 4)          # rows not whole scale tiles per rank
    with pytest.raises(ValueError):
        SlotLayout([(1024, 48)], 4)          # cols not whole MX blocks


@pytest.mark.parametrize("world,cols", [(2, 96), (4, 160), (8, 32)])
def test_a_ranks_byte_ranges_hold_exactly_the_quantisation_of_its_rows(world, cols):
    """What rank r writes (the quantisation of rows [r0, r1) alone, in the tiled scale layout of an (r1 - r0)-row matrix)
    is byte for byte what the quantisation of the whole matrix has at the byte ranges the layout gives for those rows."""
    rows = 128 * world * 2
    rng = np.random.default_rng(7 + world)
    bits = o.f32_to_bf16_bits((rng.standard_t(3, size=(rows, cols)) * 0.5).astype(np.float32))
    lay = SlotLayout([(rows, cols)], world)
    codes, sf = o.quantize_rowwise(bits)
    tiled = o.sf_flat_to_tiled(sf)
    for shared in (rows, rows // 2):
        pieces = [lay.rows_of(shared, r) for r in range(world)] + ([(shared, rows)] if shared < rows else [])
        for r0, r1 in pieces:
            c_lo, c_hi, s_lo, s_hi = lay.byte_ranges(0, r0, r1)
            part_codes, part_sf = o.quantize_rowwise(bits[r0:r1])
            assert np.array_equal(codes.reshape(-1)[c_lo:c_hi], part_codes.reshape(-1))
            assert np.array_equal(tiled.reshape(-1)[s_lo:s_hi], o.sf_flat_to_tiled(part_sf).reshape(-1))
