package cuda

// libfp8quant.so: per-tensor FP32 / FP16 -> e4m3 quantiser (include/fp8_quantize.h).  Takes the place of the
// QuantizeF32ToF8E4M3(Unit) calls of internal/abjexam/battle_a_llm.go:476-494; the amax word is cleared by the library
// on the caller's stream, so the zero-upload + Sync around each call (battle_a_llm.go:463-473) is no longer needed.
// Not compiled in the repository that ships this file (no Go toolchain there).

import (
	"fmt"
	"sync"

	"github.com/ebitengine/purego"
)

// Quantiser conventions.
const (
	FP8QuantAmaxOver448 = 0 // scale = amax / 448: codes span the e4m3 range
	FP8QuantUnit        = 1 // scale = amax: decoded magnitudes <= 1
)

var fp8quant struct {
	once      sync.Once
	err       error
	quantF32  func(x, q, scaleOut, amaxOut uintptr, n uintptr, convention int32, stream uintptr) int32
	quantFP16 func(x, q, scaleOut uintptr, n int32) int32
	dequant   func(q, out, scaleIn uintptr, n int32) int32
	sync2     func() int32
	quantMX   func(x, q, scales uintptr, rows, K int32, stream uintptr) int32
}

func initFP8Quant() error {
	fp8quant.once.Do(func() {
		lib, err := purego.Dlopen(resolveLib("libfp8quant.so"), purego.RTLD_LAZY)
		if err != nil {
			fp8quant.err = fmt.Errorf("fp8quant: dlopen: %w", err)
			return
		}
		purego.RegisterLibFunc(&fp8quant.quantF32, lib, "fp8_quantize_f32")
		purego.RegisterLibFunc(&fp8quant.quantFP16, lib, "fp8_quantize_fp16")
		purego.RegisterLibFunc(&fp8quant.dequant, lib, "fp8_dequantize_to_fp16")
		purego.RegisterLibFunc(&fp8quant.sync2, lib, "cuda_device_sync2")
		purego.RegisterLibFunc(&fp8quant.quantMX, lib, "fp8_quantize_mx_f32")
	})
	return fp8quant.err
}

func quantizeF32(src, dst, scale, amax uintptr, n int, convention int32, stream uintptr) error {
	if err := initFP8Quant(); err != nil {
		return err
	}
	if rc := fp8quant.quantF32(src, dst, scale, amax, uintptr(n), convention, stream); rc != 0 {
		return fmt.Errorf("fp8_quantize_f32: CUDA error %d", rc)
	}
	return nil
}

// QuantizeF32ToF8E4M3: codes = e4m3(x / scale), scale = amax/448 written to *scale, amax to *amax (device floats).
func QuantizeF32ToF8E4M3(src, dst, scale, amax uintptr, n int, stream uintptr) error {
	return quantizeF32(src, dst, scale, amax, n, FP8QuantAmaxOver448, stream)
}

// QuantizeF32ToF8E4M3Unit: the same with scale = amax (decoded magnitudes <= 1).
func QuantizeF32ToF8E4M3Unit(src, dst, scale, amax uintptr, n int, stream uintptr) error {
	return quantizeF32(src, dst, scale, amax, n, FP8QuantUnit, stream)
}

// QuantizeFP16: fp8_quantize_fp16 of libs1/fp8_quantize_v2.cu:176-204 (default stream, scale = amax/448).
func QuantizeFP16(src, dst, scale uintptr, n int) error {
	if err := initFP8Quant(); err != nil {
		return err
	}
	if rc := fp8quant.quantFP16(src, dst, scale, int32(n)); rc != 0 {
		return fmt.Errorf("fp8_quantize_fp16: CUDA error %d", rc)
	}
	return nil
}

// DequantizeToFP16: out[i] = fp16(decode(q[i]) * *scale).
func DequantizeToFP16(src, dst, scale uintptr, n int) error {
	if err := initFP8Quant(); err != nil {
		return err
	}
	if rc := fp8quant.dequant(src, dst, scale, int32(n)); rc != 0 {
		return fmt.Errorf("fp8_dequantize_to_fp16: CUDA error %d", rc)
	}
	return nil
}

// DeviceSync2: cuda_device_sync2.
func DeviceSync2() error {
	if err := initFP8Quant(); err != nil {
		return err
	}
	if rc := fp8quant.sync2(); rc != 0 {
		return fmt.Errorf("cuda_device_sync2: CUDA error %d", rc)
	}
	return nil
}

// QuantizeMXF32: [rows, K] fp32 -> e4m3 codes + ue8m0 block scales (one per 32 elements along K), the operand format
// of FP8GEMMMX; scales receives MXScaleBytes(rows, K) bytes.
func QuantizeMXF32(src, codes, scales uintptr, rows, K int, stream uintptr) error {
	if err := initFP8Quant(); err != nil {
		return err
	}
	if rc := fp8quant.quantMX(src, codes, scales, int32(rows), int32(K), stream); rc != 0 {
		return fmt.Errorf("fp8_quantize_mx_f32: CUDA error %d", rc)
	}
	return nil
}
