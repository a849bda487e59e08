// Thin torch-extension layer over the C ABI of libdw_mxfp8.so (module deepwell_b200._C).
//
// Same role as the reference's csrc/python_bindings.cpp: tensors in, tensors out, outputs allocated
// with the caller's options, everything on c10::cuda::getCurrentCUDAStream() (reference :88, :96,
// :211-216).  It holds no kernel and no arithmetic: every function checks its arguments, allocates
// the outputs and calls one or two entry points of include/dw_mxfp8.h.  It exists because the
// per-call cost of doing the same from Python (ctypes + several torch.empty) is larger than the GPU
// time of a GPT-2-sized linear layer.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <tuple>

#include "../../include/dw_mxfp8.h"

namespace {

using torch::Tensor;

void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == DW_OK, what, " failed: ", dw_mxfp8_error_string(rc), " (code ", rc, ")");
}

Tensor bytes_like(const Tensor& ref, std::initializer_list<int64_t> shape) {
  return torch::empty(shape, ref.options().dtype(torch::kUInt8));
}

void* stream_of(const Tensor& t) { return c10::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

const Tensor& require_bf16_2d(const Tensor& x, const char* name) {
  TORCH_CHECK(x.is_cuda(), name, " must be on CUDA");
  TORCH_CHECK(x.dim() == 2 && x.scalar_type() == torch::kBFloat16, name, " must be a 2-D bfloat16 tensor");
  return x;
}

// bf16 [rows, cols] -> (codes float8_e4m3fn, scales uint8); see dw_mxfp8_quantize
std::tuple<Tensor, Tensor> quantize(const Tensor& x_in, int64_t direction, int64_t rule, int64_t layout) {
  require_bf16_2d(x_in, "input");
  const c10::cuda::CUDAGuard guard(x_in.device());
  const Tensor x = x_in.contiguous();
  const int64_t rows = x.size(0), cols = x.size(1);
  const bool row = direction == DW_DIR_ROW;
  const int64_t op_rows = row ? rows : cols, op_k = row ? cols : rows;
  Tensor codes = direction == DW_DIR_COL_T ? bytes_like(x, {cols, rows}) : bytes_like(x, {rows, cols});
  Tensor scales = bytes_like(x, {static_cast<int64_t>(dw_mxfp8_scale_bytes(op_rows, op_k, static_cast<int>(layout)))});
  check_rc(dw_mxfp8_quantize(x.data_ptr(), codes.data_ptr(), scales.data_ptr(), rows, cols, static_cast<int>(direction),
                             static_cast<int>(rule), static_cast<int>(layout), stream_of(x)),
           "dw_mxfp8_quantize");
  if (layout == DW_SF_FLAT) scales = scales.view({op_rows, (op_k + 31) / 32});
  return {codes.view(torch::kFloat8_e4m3fn), scales};
}

// one read of x -> (codes_row, scales_row, codes_col_t, scales_col); see dw_mxfp8_quantize_both
std::tuple<Tensor, Tensor, Tensor, Tensor> quantize_both(const Tensor& x_in, int64_t rule, int64_t layout) {
  require_bf16_2d(x_in, "input");
  const c10::cuda::CUDAGuard guard(x_in.device());
  const Tensor x = x_in.contiguous();
  const int64_t rows = x.size(0), cols = x.size(1);
  Tensor cr = bytes_like(x, {rows, cols}), ct = bytes_like(x, {cols, rows});
  Tensor sr = bytes_like(x, {static_cast<int64_t>(dw_mxfp8_scale_bytes(rows, cols, static_cast<int>(layout)))});
  Tensor sc = bytes_like(x, {static_cast<int64_t>(dw_mxfp8_scale_bytes(cols, rows, static_cast<int>(layout)))});
  check_rc(dw_mxfp8_quantize_both(x.data_ptr(), cr.data_ptr(), sr.data_ptr(), ct.data_ptr(), sc.data_ptr(), rows, cols,
                                  static_cast<int>(rule), static_cast<int>(layout), stream_of(x)),
           "dw_mxfp8_quantize_both");
  if (layout == DW_SF_FLAT) {
    sr = sr.view({rows, (cols + 31) / 32});
    sc = sc.view({cols, (rows + 31) / 32});
  }
  return {cr.view(torch::kFloat8_e4m3fn), sr, ct.view(torch::kFloat8_e4m3fn), sc};
}

// dw_mxfp8_quantize_both into buffers the caller keeps (a module's persistent weight operands, so that a captured
// CUDA graph re-quantises into the addresses it recorded).  The column-wise pair may be absent.
void quantize_both_into(const Tensor& x_in, const Tensor& cr, const Tensor& sr, const c10::optional<Tensor>& ct,
                        const c10::optional<Tensor>& sc, int64_t rule) {
  require_bf16_2d(x_in, "input");
  TORCH_CHECK(x_in.is_contiguous(), "input must be contiguous");
  const c10::cuda::CUDAGuard guard(x_in.device());
  const int64_t rows = x_in.size(0), cols = x_in.size(1);
  auto check_buf = [&](const Tensor& t, int64_t bytes, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.get_device() == x_in.get_device() && t.is_contiguous() && t.element_size() == 1 &&
                    t.numel() >= bytes, name, " must be a contiguous one-byte CUDA tensor of at least ", bytes, " bytes");
  };
  check_buf(cr, rows * cols, "row codes");
  check_buf(sr, static_cast<int64_t>(dw_mxfp8_scale_bytes(rows, cols, DW_SF_TILED)), "row scales");
  TORCH_CHECK(ct.has_value() == sc.has_value(), "column codes and scales come together");
  if (ct.has_value()) {
    check_buf(*ct, rows * cols, "column codes");
    check_buf(*sc, static_cast<int64_t>(dw_mxfp8_scale_bytes(cols, rows, DW_SF_TILED)), "column scales");
  }
  check_rc(dw_mxfp8_quantize_both(x_in.data_ptr(), cr.data_ptr(), sr.data_ptr(), ct.has_value() ? ct->data_ptr() : nullptr,
                                  sc.has_value() ? sc->data_ptr() : nullptr, rows, cols, static_cast<int>(rule), DW_SF_TILED,
                                  stream_of(x_in)),
           "dw_mxfp8_quantize_both");
}

// quantize_both plus the column sums of x ([cols], fp32 or bf16); see dw_mxfp8_quantize_both_colsum
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> quantize_both_colsum(const Tensor& x_in, int64_t rule, int64_t layout,
                                                                        bool sum_bf16) {
  require_bf16_2d(x_in, "input");
  const c10::cuda::CUDAGuard guard(x_in.device());
  const Tensor x = x_in.contiguous();
  const int64_t rows = x.size(0), cols = x.size(1);
  TORCH_CHECK(rows > 0 && rows % 32 == 0 && cols > 0 && cols % 32 == 0, "rows and cols must be positive multiples of 32");
  Tensor cr = bytes_like(x, {rows, cols}), ct = bytes_like(x, {cols, rows});
  Tensor sr = bytes_like(x, {static_cast<int64_t>(dw_mxfp8_scale_bytes(rows, cols, static_cast<int>(layout)))});
  Tensor sc = bytes_like(x, {static_cast<int64_t>(dw_mxfp8_scale_bytes(cols, rows, static_cast<int>(layout)))});
  Tensor sum = torch::empty({cols}, x.options().dtype(sum_bf16 ? torch::kBFloat16 : torch::kFloat32));
  const size_t ws_bytes = dw_mxfp8_colsum_workspace(rows, cols);
  Tensor ws = bytes_like(x, {static_cast<int64_t>(ws_bytes)});
  check_rc(dw_mxfp8_quantize_both_colsum(x.data_ptr(), cr.data_ptr(), sr.data_ptr(), ct.data_ptr(), sc.data_ptr(), rows, cols,
                                         static_cast<int>(rule), static_cast<int>(layout), sum.data_ptr(), sum_bf16 ? 1 : 0,
                                         ws.data_ptr(), ws_bytes, stream_of(x)),
           "dw_mxfp8_quantize_both_colsum");
  if (layout == DW_SF_FLAT) {
    sr = sr.view({rows, (cols + 31) / 32});
    sc = sc.view({cols, (rows + 31) / 32});
  }
  return {cr.view(torch::kFloat8_e4m3fn), sr, ct.view(torch::kFloat8_e4m3fn), sc, sum};
}

// D[M,N] = alpha * A[M,K] . B[N,K]^T + beta * D + bias; operands with DW_SF_TILED scales; see dw_mxfp8_gemm.
// plan < 0: the process default (dw_mxfp8_gemm); otherwise this call's own plan word (dw_mxfp8_gemm_planned).
Tensor gemm(const Tensor& a, const Tensor& a_sf, const Tensor& b, const Tensor& b_sf, const c10::optional<Tensor>& out_in,
            const c10::optional<Tensor>& bias, double alpha, double beta, const Tensor& status, int64_t plan = -1) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a_sf.is_cuda() && b_sf.is_cuda(), "operands must be on CUDA");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.element_size() == 1 && b.element_size() == 1, "operands must be 2-D one-byte tensors");
  const int64_t M = a.size(0), K = a.size(1), N = b.size(0);
  TORCH_CHECK(b.size(1) == K, "contraction mismatch: A is [", M, ",", K, "], B is [", N, ",", b.size(1), "]");
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous(), "operands must be contiguous");
  TORCH_CHECK(a_sf.numel() >= static_cast<int64_t>(dw_mxfp8_scale_bytes(M, K, DW_SF_TILED)) &&
                  b_sf.numel() >= static_cast<int64_t>(dw_mxfp8_scale_bytes(N, K, DW_SF_TILED)),
              "scale buffers must be in the tiled (tcgen05) layout");
  const c10::cuda::CUDAGuard guard(a.device());
  Tensor out;
  if (out_in.has_value()) {
    out = *out_in;
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == torch::kBFloat16 && out.is_contiguous() && out.dim() == 2 &&
                    out.size(0) == M && out.size(1) == N,
                "out must be a contiguous bfloat16 [M, N] tensor");
  } else {
    out = torch::empty({M, N}, a.options().dtype(torch::kBFloat16));
  }
  const void* bias_ptr = nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == torch::kBFloat16 && bias->numel() == N && bias->is_contiguous(),
                "bias must be a contiguous bfloat16 [N] tensor");
    bias_ptr = bias->data_ptr();
  }
  // non-zero when the GEMM will split K
  const size_t ws_bytes = plan < 0 ? dw_mxfp8_gemm_workspace(M, N, K)
                                   : dw_mxfp8_gemm_workspace_planned(M, N, K, static_cast<int>(plan));
  Tensor ws;
  if (ws_bytes) ws = bytes_like(a, {static_cast<int64_t>(ws_bytes)});
  void* ws_ptr = ws_bytes ? ws.data_ptr() : nullptr;
  const float al = static_cast<float>(alpha), be = static_cast<float>(beta);
  if (plan < 0)
    check_rc(dw_mxfp8_gemm(a.data_ptr(), a_sf.data_ptr(), b.data_ptr(), b_sf.data_ptr(), out.data_ptr(), bias_ptr, M, N, K, al,
                           be, ws_ptr, ws_bytes, status.data_ptr(), stream_of(a)),
             "dw_mxfp8_gemm");
  else
    check_rc(dw_mxfp8_gemm_planned(a.data_ptr(), a_sf.data_ptr(), b.data_ptr(), b_sf.data_ptr(), out.data_ptr(), bias_ptr, M, N,
                                   K, al, be, ws_ptr, ws_bytes, static_cast<int>(plan), status.data_ptr(), stream_of(a)),
             "dw_mxfp8_gemm_planned");
  return out;
}

// Forward of the MXFP8 linear layer: quantise x (both forms when the weight gradient will need the
// column-wise one), GEMM against the cached row-wise weight operand, bias in the epilogue.
// Returns (y [m, N] bf16, x column-wise codes, x column-wise scales); the last two are empty tensors
// when save_col is false.  Rows are padded with zeros to a multiple of 32 for the column-wise form.
std::tuple<Tensor, Tensor, Tensor> linear_forward(const Tensor& x2d, const Tensor& w_codes, const Tensor& w_sf,
                                                  const c10::optional<Tensor>& bias, bool save_col, int64_t rule,
                                                  const Tensor& status) {
  require_bf16_2d(x2d, "input");
  const int64_t m = x2d.size(0);
  Tensor xr, xrs, xc, xcs;
  if (save_col) {
    const int64_t pad = (32 - m % 32) % 32;
    const Tensor xp = pad ? torch::constant_pad_nd(x2d, {0, 0, 0, pad}) : x2d;
    std::tie(xr, xrs, xc, xcs) = quantize_both(xp, rule, DW_SF_TILED);
  } else {
    std::tie(xr, xrs) = quantize(x2d, DW_DIR_ROW, rule, DW_SF_TILED);
  }
  Tensor y = gemm(xr, xrs, w_codes, w_sf, c10::nullopt, bias, 1.0, 0.0, status);
  if (y.size(0) != m) y = y.narrow(0, 0, m);
  return {y, xc, xcs};
}

// Backward: dX = dY . W (contraction over N, W column-wise), dW = dY^T . X (contraction over the tokens,
// both operands column-wise), db = column sums of dY (db_mode 0: not wanted, 1: bf16, 2: fp32; taken by the
// quantiser from its own read of dY when dW is wanted too).  Undefined tensors are returned for gradients that are not needed.
std::tuple<Tensor, Tensor, Tensor> linear_backward(const Tensor& dy_in, const c10::optional<Tensor>& w_col_codes,
                                                   const c10::optional<Tensor>& w_col_sf,
                                                   const c10::optional<Tensor>& x_col_codes,
                                                   const c10::optional<Tensor>& x_col_sf, int64_t m, int64_t rule,
                                                   int64_t db_mode, const Tensor& status) {
  require_bf16_2d(dy_in, "grad_output");
  const bool need_dx = w_col_codes.has_value(), need_dw = x_col_codes.has_value(), need_db = db_mode != 0;
  const int64_t pad = (32 - dy_in.size(0) % 32) % 32;
  const Tensor dy = pad ? torch::constant_pad_nd(dy_in, {0, 0, 0, pad}) : dy_in.contiguous();
  Tensor dr, drs, dc, dcs, dx, dw, db;
  if (need_dw && need_db) std::tie(dr, drs, dc, dcs, db) = quantize_both_colsum(dy, rule, DW_SF_TILED, db_mode == 1);
  else if (need_dw) std::tie(dr, drs, dc, dcs) = quantize_both(dy, rule, DW_SF_TILED);
  else if (need_dx) std::tie(dr, drs) = quantize(dy, DW_DIR_ROW, rule, DW_SF_TILED);
  if (need_db && !db.defined()) db = db_mode == 1 ? dy_in.sum({0}) : dy_in.sum({0}, false, torch::kFloat32);
  if (need_dx) {
    dx = gemm(dr, drs, *w_col_codes, *w_col_sf, c10::nullopt, c10::nullopt, 1.0, 0.0, status);
    if (dx.size(0) != m) dx = dx.narrow(0, 0, m);
  }
  if (need_dw) dw = gemm(dc, dcs, *x_col_codes, *x_col_sf, c10::nullopt, c10::nullopt, 1.0, 0.0, status);
  return {dx, dw, db};
}

// The linear layer as one autograd node: forward and backward above, with the quantised operands the backward needs
// (the column-wise form of x for the weight gradient, of W for the input gradient) carried in the node.  `weight` takes
// part only so that autograd asks for its gradient; the arithmetic reads the quantised operands the caller keeps.
// Having the node here rather than in Python keeps the interpreter out of the backward pass (a GPT-2-sized layer's
// kernels take less time than a Python-level backward costs).
class MXFP8LinearFunction : public torch::autograd::Function<MXFP8LinearFunction> {
 public:
  static Tensor forward(torch::autograd::AutogradContext* ctx, const Tensor& x2d, const Tensor& weight,
                        const c10::optional<Tensor>& bias, const Tensor& w_row_codes, const Tensor& w_row_sf,
                        const c10::optional<Tensor>& w_col_codes, const c10::optional<Tensor>& w_col_sf, int64_t rule,
                        const Tensor& status, bool check_status, bool need_dx, bool need_dw) {
    // need_dx / need_dw come from the caller: inside forward() gradient mode is switched off
    TORCH_CHECK(!need_dx || w_col_codes.has_value(), "the input gradient needs the column-wise weight operand");
    const Tensor xb = x2d.scalar_type() == torch::kBFloat16 ? x2d : x2d.to(torch::kBFloat16);
    c10::optional<Tensor> bias_b;
    if (bias.has_value() && bias->defined())
      bias_b = bias->scalar_type() == torch::kBFloat16 ? *bias : bias->to(torch::kBFloat16);
    Tensor y, xc, xcs;
    std::tie(y, xc, xcs) = linear_forward(xb.detach(), w_row_codes, w_row_sf, bias_b, need_dw, rule, status);
    ctx->saved_data["m"] = xb.size(0);
    ctx->saved_data["rule"] = rule;
    ctx->saved_data["status"] = status;
    ctx->saved_data["check_status"] = check_status;
    ctx->saved_data["x_dtype"] = static_cast<int64_t>(x2d.scalar_type());
    ctx->saved_data["w_dtype"] = static_cast<int64_t>(weight.scalar_type());
    ctx->saved_data["bias_dtype"] = bias_b.has_value() ? static_cast<int64_t>(bias->scalar_type()) : int64_t(-1);
    if (need_dw) {
      ctx->saved_data["x_col_codes"] = xc;
      ctx->saved_data["x_col_sf"] = xcs;
    }
    if (need_dx) {
      ctx->saved_data["w_col_codes"] = *w_col_codes;
      ctx->saved_data["w_col_sf"] = *w_col_sf;
    }
    return x2d.scalar_type() == torch::kBFloat16 ? y : y.to(x2d.scalar_type());
  }

  static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::variable_list grad_outputs) {
    const Tensor& dy_in = grad_outputs[0];
    const bool need_dx = ctx->needs_input_grad(0) && ctx->saved_data.count("w_col_codes") > 0;
    const bool need_dw = ctx->needs_input_grad(1) && ctx->saved_data.count("x_col_codes") > 0;
    const int64_t bias_dtype = ctx->saved_data["bias_dtype"].toInt();
    const bool need_db = ctx->needs_input_grad(2) && bias_dtype >= 0;
    const Tensor dy = dy_in.scalar_type() == torch::kBFloat16 ? dy_in : dy_in.to(torch::kBFloat16);
    c10::optional<Tensor> w_cc, w_cs, x_cc, x_cs;
    if (need_dx) { w_cc = ctx->saved_data["w_col_codes"].toTensor(); w_cs = ctx->saved_data["w_col_sf"].toTensor(); }
    if (need_dw) { x_cc = ctx->saved_data["x_col_codes"].toTensor(); x_cs = ctx->saved_data["x_col_sf"].toTensor(); }
    // bf16 column sums only for a bf16 bias; fp32 sums otherwise
    const int64_t db_mode = !need_db ? 0 : (bias_dtype == static_cast<int64_t>(torch::kBFloat16) ? 1 : 2);
    const Tensor status = ctx->saved_data["status"].toTensor();
    Tensor dx, dw, db;
    std::tie(dx, dw, db) = linear_backward(dy, w_cc, w_cs, x_cc, x_cs, ctx->saved_data["m"].toInt(),
                                           ctx->saved_data["rule"].toInt(), db_mode, status);
    const auto x_dtype = static_cast<torch::ScalarType>(ctx->saved_data["x_dtype"].toInt());
    const auto w_dtype = static_cast<torch::ScalarType>(ctx->saved_data["w_dtype"].toInt());
    if (dx.defined() && dx.scalar_type() != x_dtype) dx = dx.to(x_dtype);
    if (dw.defined() && dw.scalar_type() != w_dtype) dw = dw.to(w_dtype);
    if (db.defined() && bias_dtype >= 0 && db.scalar_type() != static_cast<torch::ScalarType>(bias_dtype))
      db = db.to(static_cast<torch::ScalarType>(bias_dtype));
    if (ctx->saved_data["check_status"].toBool()) {
      const c10::cuda::CUDAGuard guard(dy.device());
      check_rc(dw_mxfp8_check_status(status.data_ptr(), stream_of(dy)), "DWLinear backward");
    }
    return {dx, dw, db, Tensor(), Tensor(), Tensor(), Tensor(), Tensor(), Tensor(), Tensor(), Tensor(), Tensor()};
  }
};

// y = x2d . W^T + bias with gradients (see MXFP8LinearFunction); the weight's quantised operands come from the caller.
Tensor linear(const Tensor& x2d, const Tensor& weight, const c10::optional<Tensor>& bias, const Tensor& w_row_codes,
              const Tensor& w_row_sf, const c10::optional<Tensor>& w_col_codes, const c10::optional<Tensor>& w_col_sf,
              int64_t rule, const Tensor& status, bool check_status) {
  const bool grad_mode = c10::GradMode::is_enabled();
  return MXFP8LinearFunction::apply(x2d, weight, bias, w_row_codes, w_row_sf, w_col_codes, w_col_sf, rule, status,
                                    check_status, grad_mode && x2d.requires_grad(), grad_mode && weight.requires_grad());
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "torch-tensor layer over libdw_mxfp8.so (MX quantisation + block-scaled GEMM for sm_100a)";
  m.def("quantize", &quantize, py::arg("x"), py::arg("direction"), py::arg("rule"), py::arg("layout"));
  m.def("quantize_both", &quantize_both, py::arg("x"), py::arg("rule"), py::arg("layout"));
  m.def("quantize_both_into", &quantize_both_into, py::arg("x"), py::arg("codes_row"), py::arg("scales_row"),
        py::arg("codes_col_t") = py::none(), py::arg("scales_col") = py::none(), py::arg("rule") = 0);
  m.def("quantize_both_colsum", &quantize_both_colsum, py::arg("x"), py::arg("rule"), py::arg("layout"), py::arg("sum_bf16"));
  m.def("gemm", &gemm, py::arg("a"), py::arg("a_sf"), py::arg("b"), py::arg("b_sf"), py::arg("out") = py::none(),
        py::arg("bias") = py::none(), py::arg("alpha") = 1.0, py::arg("beta") = 0.0, py::arg("status"), py::arg("plan") = -1);
  m.def("linear", &linear, py::arg("x2d"), py::arg("weight"), py::arg("bias"), py::arg("w_row_codes"), py::arg("w_row_sf"),
        py::arg("w_col_codes"), py::arg("w_col_sf"), py::arg("rule"), py::arg("status"), py::arg("check_status") = false);
  m.def("linear_forward", &linear_forward);
  m.def("linear_backward", &linear_backward);
}
