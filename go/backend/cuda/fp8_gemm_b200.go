package cuda

// Additive entry points of the sm_100a libfp8gemm.so (include/fp8_gemm.h).  The three reference symbols stay bound
// in fp8_gemm.go; these are registered against the same library handle.  Not compiled in the repository that ships
// this file (no Go toolchain there): it mirrors goml_b200/host/goml_cuda.hpp call for call.

import (
	"fmt"
	"sync"

	"github.com/ebitengine/purego"
)

// Output types of FP8GEMMScaled.
const (
	FP8OutFP16 = 0
	FP8OutBF16 = 1
)

var fp8gemmB200 struct {
	once     sync.Once
	err      error
	scaled   func(M, N, K int32, A, B, C uintptr, alpha float32, scaleA, scaleB uintptr, outDType int32, stream uintptr) int32
	accF32   func(M, N, K int32, A, B, X uintptr, alpha float32, scaleA, scaleB, stream uintptr) int32
	swiglu   func(M, F, K int32, A, Binterleaved, H uintptr, alpha float32, scaleA, scaleB, amaxOut, stream uintptr) int32
	fp8out   func(M, N, K int32, A, B, D uintptr, alpha float32, scaleA, scaleB, scaleD, amaxD, stream uintptr) int32
	status   func() int32
	setPairs func(mode int32) int32
	mx       func(M, N, K int32, A, scaleA, B, scaleB, C uintptr, alpha float32, outDType int32, stream uintptr) int32
	mxBytes  func(rows, K int32) uintptr
}

func initFP8GEMMB200() error {
	if err := initFP8GEMM(); err != nil { // dlopen + the three reference symbols (fp8_gemm.go)
		return err
	}
	fp8gemmB200.once.Do(func() {
		defer func() {
			if r := recover(); r != nil { // RegisterLibFunc panics on a missing symbol: an older library
				fp8gemmB200.err = fmt.Errorf("fp8gemm: library lacks the sm_100a extensions: %v", r)
			}
		}()
		lib := fp8gemm.lib
		purego.RegisterLibFunc(&fp8gemmB200.scaled, lib, "fp8_gemm_scaled")
		purego.RegisterLibFunc(&fp8gemmB200.accF32, lib, "fp8_gemm_accumulate_f32")
		purego.RegisterLibFunc(&fp8gemmB200.swiglu, lib, "fp8_gemm_swiglu")
		purego.RegisterLibFunc(&fp8gemmB200.fp8out, lib, "fp8_gemm_fp8out")
		purego.RegisterLibFunc(&fp8gemmB200.status, lib, "fp8_gemm_device_status")
		purego.RegisterLibFunc(&fp8gemmB200.setPairs, lib, "fp8_gemm_set_tile_pairs")
		purego.RegisterLibFunc(&fp8gemmB200.mx, lib, "fp8_gemm_mx")
		purego.RegisterLibFunc(&fp8gemmB200.mxBytes, lib, "fp8_mx_scale_bytes")
	})
	return fp8gemmB200.err
}

// FP8GEMMScaled: C = alpha * (*scaleA) * (*scaleB) * A x B^T.  scaleA / scaleB are device pointers to one float each
// (what the quantiser wrote) or 0; outDType is FP8OutFP16 or FP8OutBF16.
func FP8GEMMScaled(M, N, K int, A, B, C uintptr, alpha float32, scaleA, scaleB uintptr, outDType int, stream uintptr) error {
	if err := initFP8GEMMB200(); err != nil {
		return err
	}
	if rc := fp8gemmB200.scaled(int32(M), int32(N), int32(K), A, B, C, alpha, scaleA, scaleB, int32(outDType), stream); rc != 0 {
		return fmt.Errorf("fp8_gemm_scaled: CUDA error %d", rc)
	}
	return nil
}

// FP8GEMMAccumulateF32: X (fp32 [M,N]) += alpha * sa * sb * A x B^T — a decoder block's residual update in the epilogue.
func FP8GEMMAccumulateF32(M, N, K int, A, B, X uintptr, alpha float32, scaleA, scaleB, stream uintptr) error {
	if err := initFP8GEMMB200(); err != nil {
		return err
	}
	if rc := fp8gemmB200.accF32(int32(M), int32(N), int32(K), A, B, X, alpha, scaleA, scaleB, stream); rc != 0 {
		return fmt.Errorf("fp8_gemm_accumulate_f32: CUDA error %d", rc)
	}
	return nil
}

// FP8GEMMSwiGLU: H (bf16 [M,F]) = silu(g) * u with [g | u] from the interleaved gate/up weight; max|H| -> *amaxOut.
func FP8GEMMSwiGLU(M, F, K int, A, Binterleaved, H uintptr, alpha float32, scaleA, scaleB, amaxOut, stream uintptr) error {
	if err := initFP8GEMMB200(); err != nil {
		return err
	}
	if rc := fp8gemmB200.swiglu(int32(M), int32(F), int32(K), A, Binterleaved, H, alpha, scaleA, scaleB, amaxOut, stream); rc != 0 {
		return fmt.Errorf("fp8_gemm_swiglu: CUDA error %d", rc)
	}
	return nil
}

// FP8GEMMFP8Out: D (e4m3) = e4m3((*scaleD) * v), v = alpha * sa * sb * A x B^T, max|v| -> *amaxD (0: not wanted).
func FP8GEMMFP8Out(M, N, K int, A, B, D uintptr, alpha float32, scaleA, scaleB, scaleD, amaxD, stream uintptr) error {
	if err := initFP8GEMMB200(); err != nil {
		return err
	}
	if rc := fp8gemmB200.fp8out(int32(M), int32(N), int32(K), A, B, D, alpha, scaleA, scaleB, scaleD, amaxD, stream); rc != 0 {
		return fmt.Errorf("fp8_gemm_fp8out: CUDA error %d", rc)
	}
	return nil
}

// InterleaveGateUp lays a [2F, K] gate-then-up weight (e4m3 codes, host memory) out the way FP8GEMMSwiGLU reads it:
// per 32 feed-forward columns the 32 gate rows followed by the 32 up rows; rows past F (F rounded up to 32) are zero.
func InterleaveGateUp(w []byte, F, K int) []byte {
	Fp := (F + 31) / 32 * 32
	out := make([]byte, 2*Fp*K)
	for f := 0; f < F; f++ {
		blk, r := f/32, f%32
		copy(out[((blk*2)*32+r)*K:], w[f*K:(f+1)*K])       // gate row f
		copy(out[((blk*2+1)*32+r)*K:], w[(F+f)*K:(F+f+1)*K]) // up row f
	}
	return out
}

// FP8GEMMDeviceStatus synchronises the current device and returns (and clears) the code a GEMM kernel recorded when
// one of its bounded waits ran out; 0 in normal operation.
func FP8GEMMDeviceStatus() (int, error) {
	if err := initFP8GEMMB200(); err != nil {
		return 0, err
	}
	rc := int(fp8gemmB200.status())
	if rc < 0 {
		return 0, fmt.Errorf("fp8_gemm_device_status: CUDA error %d", -rc)
	}
	return rc, nil
}

// FP8GEMMSetTilePairs: -1 = tile pairs chosen per problem (default), 0 = single tiles only (bit-identical results).
func FP8GEMMSetTilePairs(mode int) error {
	if err := initFP8GEMMB200(); err != nil {
		return err
	}
	if rc := fp8gemmB200.setPairs(int32(mode)); rc != 0 {
		return fmt.Errorf("fp8_gemm_set_tile_pairs: CUDA error %d", rc)
	}
	return nil
}

// FP8GEMMMX: the block-scaled ("MXFP8") GEMM — e4m3 codes with one ue8m0 scale per 32 K elements of every row of A and
// of B (the arrays QuantizeMXF32 writes); C = alpha * sum over blocks of 2^(ea+eb) * A_kb . B_kb.  K % 128 == 0.
func FP8GEMMMX(M, N, K int, A, scaleA, B, scaleB, C uintptr, alpha float32, outDType int, stream uintptr) error {
	if err := initFP8GEMMB200(); err != nil {
		return err
	}
	if rc := fp8gemmB200.mx(int32(M), int32(N), int32(K), A, scaleA, B, scaleB, C, alpha, int32(outDType), stream); rc != 0 {
		return fmt.Errorf("fp8_gemm_mx: CUDA error %d", rc)
	}
	return nil
}

// MXScaleBytes: size of the tiled scale array of a [rows, K] block-scaled tensor.
func MXScaleBytes(rows, K int) (int, error) {
	if err := initFP8GEMMB200(); err != nil {
		return 0, err
	}
	return int(fp8gemmB200.mxBytes(int32(rows), int32(K))), nil
}
