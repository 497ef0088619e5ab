package cuda

// libfp8block.so: the decoder block's row-local glue fused with the quantiser of the next FP8 operand
// (include/fp8_block.h).  Takes the place of rmsnorm_forward / rope_forward / swiglu_forward of libtransformer.so
// (libs/transformer_kernels.cu:384-438) followed by a quantiser launch each, and of the host round trips of
// internal/abjexam/battle_a_llm.go:380-494.  Not compiled in the repository that ships this file (no Go toolchain there).

import (
	"fmt"
	"sync"

	"github.com/ebitengine/purego"
)

// FP8DecodeAppendArgs mirrors fp8_decode_append_args_t, C layout.
type FP8DecodeAppendArgs struct {
	QKVBF16, CosTab, SinTab, Positions uintptr
	QOut, QScaleOut, QAmaxOut          uintptr
	KCache, VCache, KScale, VScale     uintptr
	SeqLensOut, BlockTable             uintptr
	Batch, QHeads, KVHeads, HeadDim    int32
	SMax, RopeRows                     int32
	PageSize, MaxPagesPerSeq, NumPages int32
	Reserved                           int32
	Stream                             uintptr
}

var fp8block struct {
	once           sync.Once
	err            error
	ropeTable      func(cos, sin uintptr, seqLen, headDim int32, theta float32, stream uintptr) int32
	rmsnormQuant   func(x, residualBF16, hOut, gamma, q, scale, amax, rstdWs uintptr, rows, hidden int32, eps float32, stream uintptr) int32
	ropeQuantQKV   func(qkvBF16, cos, sin, q, k, v, scales, amaxes uintptr, batch, seqLen, heads, headDim int32, stream uintptr) int32
	permuteQuant   func(oFP16, q, scale, amax uintptr, batch, seqLen, heads, headDim int32, stream uintptr) int32
	swigluQuant    func(gateUpBF16, q, scale, amax uintptr, rows, ffnHidden int32, stream uintptr) int32
	quantBF16      func(xBF16, q, scale, amaxIn uintptr, n uintptr, stream uintptr) int32
	residualAdd    func(x, yBF16 uintptr, n uintptr, stream uintptr) int32
	decodeRopeAppd func(args *FP8DecodeAppendArgs) int32
}

func initFP8Block() error {
	fp8block.once.Do(func() {
		lib, err := purego.Dlopen(resolveLib("libfp8block.so"), purego.RTLD_LAZY)
		if err != nil {
			fp8block.err = fmt.Errorf("fp8block: dlopen: %w", err)
			return
		}
		purego.RegisterLibFunc(&fp8block.ropeTable, lib, "fp8_rope_table")
		purego.RegisterLibFunc(&fp8block.rmsnormQuant, lib, "fp8_rmsnorm_quantize")
		purego.RegisterLibFunc(&fp8block.ropeQuantQKV, lib, "fp8_rope_quantize_qkv")
		purego.RegisterLibFunc(&fp8block.permuteQuant, lib, "fp8_permute_quantize_heads")
		purego.RegisterLibFunc(&fp8block.swigluQuant, lib, "fp8_swiglu_quantize")
		purego.RegisterLibFunc(&fp8block.quantBF16, lib, "fp8_quantize_bf16")
		purego.RegisterLibFunc(&fp8block.residualAdd, lib, "fp8_residual_add")
		purego.RegisterLibFunc(&fp8block.decodeRopeAppd, lib, "fp8_decode_rope_append")
	})
	return fp8block.err
}

func blockErr(name string, rc int32) error {
	if rc != 0 {
		return fmt.Errorf("%s: CUDA error %d", name, rc)
	}
	return nil
}

// FP8RopeTable fills cos/sin [seqLen, headDim/2] (fp32) for half-split RoPE with base theta.
func FP8RopeTable(cos, sin uintptr, seqLen, headDim int, theta float32, stream uintptr) error {
	if err := initFP8Block(); err != nil {
		return err
	}
	return blockErr("fp8_rope_table", fp8block.ropeTable(cos, sin, int32(seqLen), int32(headDim), theta, stream))
}

// FP8RMSNormQuantize: h = x (+ residual, written to hOut when given); codes of (h*gamma)*rstd with one scale.
func FP8RMSNormQuantize(x, residualBF16, hOut, gamma, q, scale, amax, rstdWs uintptr, rows, hidden int, eps float32, stream uintptr) error {
	if err := initFP8Block(); err != nil {
		return err
	}
	return blockErr("fp8_rmsnorm_quantize", fp8block.rmsnormQuant(x, residualBF16, hOut, gamma, q, scale, amax, rstdWs, int32(rows), int32(hidden), eps, stream))
}

// FP8RopeQuantizeQKV: [T,3,H,hd] bf16 projection -> RoPE on Q and K -> three [B*H,S,hd] code tensors; scales / amaxes
// are three floats each (Q, K, V order) — the pointers FAForwardArgs.ScaleQDev/KDev/VDev take.
func FP8RopeQuantizeQKV(qkvBF16, cos, sin, q, k, v, scales, amaxes uintptr, batch, seqLen, heads, headDim int, stream uintptr) error {
	if err := initFP8Block(); err != nil {
		return err
	}
	return blockErr("fp8_rope_quantize_qkv", fp8block.ropeQuantQKV(qkvBF16, cos, sin, q, k, v, scales, amaxes, int32(batch), int32(seqLen), int32(heads), int32(headDim), stream))
}

// FP8PermuteQuantizeHeads: attention output [B*H,S,hd] fp16 -> token-major codes [B*S, H*hd].
func FP8PermuteQuantizeHeads(oFP16, q, scale, amax uintptr, batch, seqLen, heads, headDim int, stream uintptr) error {
	if err := initFP8Block(); err != nil {
		return err
	}
	return blockErr("fp8_permute_quantize_heads", fp8block.permuteQuant(oFP16, q, scale, amax, int32(batch), int32(seqLen), int32(heads), int32(headDim), stream))
}

// FP8SwiGLUQuantize: [rows, 2F] bf16 gate|up -> codes of silu(gate)*up (for callers that keep a 16-bit gate/up matrix).
func FP8SwiGLUQuantize(gateUpBF16, q, scale, amax uintptr, rows, ffnHidden int, stream uintptr) error {
	if err := initFP8Block(); err != nil {
		return err
	}
	return blockErr("fp8_swiglu_quantize", fp8block.swigluQuant(gateUpBF16, q, scale, amax, int32(rows), int32(ffnHidden), stream))
}

// FP8QuantizeBF16: one pass over a bf16 tensor whose amax the producer already reduced (FP8GEMMSwiGLU's amaxOut).
func FP8QuantizeBF16(xBF16, q, scale, amaxIn uintptr, n int, stream uintptr) error {
	if err := initFP8Block(); err != nil {
		return err
	}
	return blockErr("fp8_quantize_bf16", fp8block.quantBF16(xBF16, q, scale, amaxIn, uintptr(n), stream))
}

// FP8ResidualAdd: x (fp32) += y (bf16).
func FP8ResidualAdd(x, yBF16 uintptr, n int, stream uintptr) error {
	if err := initFP8Block(); err != nil {
		return err
	}
	return blockErr("fp8_residual_add", fp8block.residualAdd(x, yBF16, uintptr(n), stream))
}

// FP8DecodeRopeAppend: the new token of every sequence — RoPE at its position, Q codes with a fresh scale, K/V codes
// with the cache's scales written into the contiguous or paged cache, lengths advanced.
func FP8DecodeRopeAppend(a *FP8DecodeAppendArgs) error {
	if err := initFP8Block(); err != nil {
		return err
	}
	return blockErr("fp8_decode_rope_append", fp8block.decodeRopeAppd(a))
}
