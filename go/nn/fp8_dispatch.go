package nn

// FP8 dispatch of the nn call sites on a B200: the device-side sequence Linear.Forward (nn/linear.go:53-74),
// FeedForward.forwardSwiGLU (nn/feedforward.go:54-79) and MultiHeadAttention.Forward (nn/attention.go:60-160) take when
// the weights have FP8 copies and the activations live on the GPU.  goml has no such path today (both run in F32
// through ops.MatMul / ops.ScaledDotProductAttention); these functions work on raw device buffers, like the chain in
// internal/abjexam/battle_a_llm.go:335-679, and leave tensor bookkeeping to the caller.
//
// Not compiled in the repository that ships this file (no Go toolchain there).  FP8DecoderBlock.Forward issues,
// call for call, what goml_b200/nn.py: FP8DecoderBlock.forward_fused issues; that Python twin is what the parity
// tests run against the CPU restatement of internal/abjexam/llama_hf_f64ref.go:94-178.

import (
	"math"

	"github.com/djeday123/goml/backend/cuda"
)

// FP8Tensor is a tensor of e4m3 codes on the device with its per-tensor scale and amax (one float each, on the device).
type FP8Tensor struct {
	Codes       uintptr
	Scale, Amax uintptr
}

// FP8Linear holds a weight [out, in] quantised once (scale = amax/448).
type FP8Linear struct {
	In, Out int
	W       FP8Tensor
}

// Forward: y (bf16 [M, Out]) = x W^T for an activation that is already e4m3 codes with a device scale.
func (l *FP8Linear) Forward(x FP8Tensor, M int, y uintptr, stream uintptr) error {
	return cuda.FP8GEMMScaled(M, l.Out, l.In, x.Codes, l.W.Codes, y, 1.0, x.Scale, l.W.Scale, cuda.FP8OutBF16, stream)
}

// AccumulateInto: h (fp32 [M, Out]) += x W^T, added in the GEMM epilogue (a residual update without a 16-bit intermediate).
func (l *FP8Linear) AccumulateInto(x FP8Tensor, M int, h uintptr, stream uintptr) error {
	return cuda.FP8GEMMAccumulateF32(M, l.Out, l.In, x.Codes, l.W.Codes, h, 1.0, x.Scale, l.W.Scale, stream)
}

// FP8Attention: O = softmax(Q K^T / sqrt(hd)) V on per-tensor quantised Q, K, V laid out [B*H, S, hd]; the three scales
// stay on the device (scales points at three consecutive floats: Q, K, V), so there is no host round trip between the
// quantiser and the attention and O comes out in real units.
func FP8Attention(fa *cuda.FAContext, q, k, v, o, lse, scales uintptr, bh, sl, hd int, causal bool, stream uintptr) error {
	c := int32(0)
	if causal {
		c = 1
	}
	return fa.ForwardEx(&cuda.FAForwardArgs{
		Q: q, K: k, V: v, O: o, LOut: lse,
		BatchHeads: int32(bh), SeqLen: int32(sl), HeadDim: int32(hd), Causal: c,
		Scale: float32(1.0 / math.Sqrt(float64(hd))), VDescale: 1.0,
		ScaleQDev: scales, ScaleKDev: scales + 4, ScaleVDev: scales + 8, Stream: stream,
	})
}

// BlockBuffers are the device buffers one prefill pass of a block needs; the caller allocates them once per shape.
type BlockBuffers struct {
	Rstd                uintptr   // fp32 [T]
	XQ, OQ, HQ          FP8Tensor // [T, d], [T, d], [T, F]
	QKV                 uintptr   // bf16 [T, 3, H, hd]
	Qc, Kc, Vc          uintptr   // e4m3 [B*H, S, hd]
	QKVScales, QKVAmax  uintptr   // 3 floats each
	O                   uintptr   // fp16 [B*H, S, hd]
	Hb                  uintptr   // bf16 [T, F]
	Cos, Sin            uintptr   // fp32 [S, hd/2], filled by cuda.FP8RopeTable
}

// FP8DecoderBlock is a Llama-style block (RMSNorm, QKV, half-split RoPE, causal attention, O, residual, RMSNorm,
// SwiGLU, residual) with every GEMM and the attention in FP8.
type FP8DecoderBlock struct {
	D, H, F            int
	Eps                float32
	QKV, O, Down       FP8Linear
	GateUpInterleaved  FP8Tensor // [2*Fp, d] in the layout cuda.InterleaveGateUp produces
	Norm1, Norm2       uintptr   // fp32 [d]
	FA                 *cuda.FAContext
}

// Forward updates the fp32 residual stream h [B*S, d] in place: ten library calls, no host synchronisation.
func (b *FP8DecoderBlock) Forward(h uintptr, B, S int, w *BlockBuffers, stream uintptr) error {
	T, hd := B*S, b.D/b.H
	// attention half
	if err := cuda.FP8RMSNormQuantize(h, 0, 0, b.Norm1, w.XQ.Codes, w.XQ.Scale, w.XQ.Amax, w.Rstd, T, b.D, b.Eps, stream); err != nil {
		return err
	}
	if err := b.QKV.Forward(w.XQ, T, w.QKV, stream); err != nil {
		return err
	}
	if err := cuda.FP8RopeQuantizeQKV(w.QKV, w.Cos, w.Sin, w.Qc, w.Kc, w.Vc, w.QKVScales, w.QKVAmax, B, S, b.H, hd, stream); err != nil {
		return err
	}
	if err := FP8Attention(b.FA, w.Qc, w.Kc, w.Vc, w.O, 0, w.QKVScales, B*b.H, S, hd, true, stream); err != nil {
		return err
	}
	if err := cuda.FP8PermuteQuantizeHeads(w.O, w.OQ.Codes, w.OQ.Scale, w.OQ.Amax, B, S, b.H, hd, stream); err != nil {
		return err
	}
	if err := b.O.AccumulateInto(w.OQ, T, h, stream); err != nil { // h += attention projection
		return err
	}
	// feed-forward half
	if err := cuda.FP8RMSNormQuantize(h, 0, 0, b.Norm2, w.XQ.Codes, w.XQ.Scale, w.XQ.Amax, w.Rstd, T, b.D, b.Eps, stream); err != nil {
		return err
	}
	if err := cuda.FP8GEMMSwiGLU(T, b.F, b.D, w.XQ.Codes, b.GateUpInterleaved.Codes, w.Hb, 1.0, w.XQ.Scale, b.GateUpInterleaved.Scale, w.HQ.Amax, stream); err != nil {
		return err
	}
	if err := cuda.FP8QuantizeBF16(w.Hb, w.HQ.Codes, w.HQ.Scale, w.HQ.Amax, T*b.F, stream); err != nil {
		return err
	}
	return b.Down.AccumulateInto(w.HQ, T, h, stream) // h += feed-forward output
}
