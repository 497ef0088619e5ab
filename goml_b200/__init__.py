"""goml_b200 — B200 (sm_100a) FP8 attention-forward and FP8 GEMM behind goml's C ABI.

Host-side mirror of the reference's ``backend/cuda`` bindings for this path:
``loader`` (arch.go), ``fp8_gemm`` (fp8_gemm.go), ``fa_forward`` (fa_forward.go).
The compute lives in the shared libraries under ``goml_b200/libs`` built from
``goml_b200/csrc`` by ``goml_b200.build``; there is no CPU fallback.
"""
__version__ = "1.0.0"
