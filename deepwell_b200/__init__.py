"""deepwell_b200 — B200 (sm_100a) implementation of Deepwell's MXFP8 linear path."""
__version__ = "0.1.0"
