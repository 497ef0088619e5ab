package cuda

// Additive entry points of the sm_100a libfa_sm120.so (include/fa_sm120.h): the struct-pointer forward (V descale and
// device-side scales), the forward that allocates nothing, the decode step, and the device status reads.  FALoad,
// FACreate, ForwardTrain and FAVersion stay in fa_forward.go.  Not compiled in the repository that ships this file (no
// Go toolchain there): it mirrors goml_b200/host/goml_cuda.hpp call for call.

import (
	"fmt"
	"runtime"
	"sync"

	"github.com/ebitengine/purego"
)

// FAForwardArgs mirrors fa_forward_args_t, C layout (104 bytes).
type FAForwardArgs struct {
	Q, K, V, O, LOut                uintptr // LOut: fp32 [bh, sl] or 0
	BatchHeads, SeqLen, HeadDim     int32
	Causal, Window                  int32
	Scale, VDescale                 float32 // VDescale 0 is treated as 1
	_                               int32   // padding before the 8-byte pointers below
	ScaleQDev, ScaleKDev, ScaleVDev uintptr // device pointers to one float each, or 0
	Stream                          uintptr
}

// FADecodeArgs mirrors fa_decode_args_t, C layout.
type FADecodeArgs struct {
	Q, KCache, VCache, O, LOut, SeqLens uintptr // SeqLens: batch int32 lengths on the device, or 0
	Batch, QHeads, KVHeads, HeadDim     int32
	SMax, SeqLen                        int32 // cache rows per head; common length when SeqLens == 0
	Scale, VDescale                     float32
	ScaleQDev, ScaleKDev, ScaleVDev     uintptr
	Stream                              uintptr
	BlockTable                          uintptr // 0: contiguous cache; else int32 [batch, MaxPagesPerSeq] on the device
	PageSize, MaxPagesPerSeq, NumPages  int32   // paged: pools [NumPages, KVHeads, PageSize, HeadDim], PageSize % 64 == 0
	_                                   int32   // C tail padding
}

var faB200 struct {
	once          sync.Once
	err           error
	forwardEx     func(ctx uintptr, args *FAForwardArgs) int32
	forwardNoAll  func(args *FAForwardArgs, errBuf *byte, errLen int32) int32
	decode        func(ctx uintptr, args *FADecodeArgs) int32
	deviceStatus  func(ctx uintptr) int32
	noAllocStatus func() int32
}

func initFAB200() error {
	if err := FALoad(); err != nil {
		return err
	}
	faB200.once.Do(func() {
		defer func() {
			if r := recover(); r != nil {
				faB200.err = fmt.Errorf("fa: library lacks the sm_100a extensions: %v", r)
			}
		}()
		purego.RegisterLibFunc(&faB200.forwardEx, faLib, "fa_forward_ex")
		purego.RegisterLibFunc(&faB200.forwardNoAll, faLib, "fa_forward_noalloc")
		purego.RegisterLibFunc(&faB200.decode, faLib, "fa_decode")
		purego.RegisterLibFunc(&faB200.deviceStatus, faLib, "fa_device_status")
		purego.RegisterLibFunc(&faB200.noAllocStatus, faLib, "fa_noalloc_device_status")
	})
	return faB200.err
}

// ForwardEx: fa_forward_ex.  With ScaleQDev/ScaleKDev/ScaleVDev set to the floats the quantiser wrote, the chain
// quantise -> attention needs no host round trip, and O comes out in real units (no host-side multiply by scaleV).
func (c *FAContext) ForwardEx(a *FAForwardArgs) error {
	if c == nil || c.ptr == 0 {
		return fmt.Errorf("FAContext.ForwardEx: nil ctx")
	}
	if err := initFAB200(); err != nil {
		return err
	}
	runtime.LockOSThread() // the C side uses the calling thread's current device
	defer runtime.UnlockOSThread()
	if st := FAStatus(faB200.forwardEx(c.ptr, a)); st != FA_OK {
		return fmt.Errorf("fa_forward_ex: %s (%s)", st, cString(faLastErr(c.ptr)))
	}
	return nil
}

// FAForwardNoAlloc: fa_forward_noalloc, for processes that may not call the allocator after start-up.  No context;
// the scratch is a fixed 32 MiB array inside the library, so BatchHeads*SeqLen*HeadDim <= 16 Mi per call.  Calls that
// overlap on the GPU share that array: keep them on one stream.  Make the first call during start-up.
func FAForwardNoAlloc(a *FAForwardArgs) error {
	if err := initFAB200(); err != nil {
		return err
	}
	runtime.LockOSThread()
	defer runtime.UnlockOSThread()
	var buf [256]byte
	if st := FAStatus(faB200.forwardNoAll(a, &buf[0], int32(len(buf)))); st != FA_OK {
		n := 0
		for n < len(buf) && buf[n] != 0 {
			n++
		}
		return fmt.Errorf("fa_forward_noalloc: %s (%s)", st, string(buf[:n]))
	}
	return nil
}

// Decode: fa_decode — one new token per sequence against an FP8 KV cache, grouped-query heads.
func (c *FAContext) Decode(a *FADecodeArgs) error {
	if c == nil || c.ptr == 0 {
		return fmt.Errorf("FAContext.Decode: nil ctx")
	}
	if err := initFAB200(); err != nil {
		return err
	}
	runtime.LockOSThread()
	defer runtime.UnlockOSThread()
	if st := FAStatus(faB200.decode(c.ptr, a)); st != FA_OK {
		return fmt.Errorf("fa_decode: %s (%s)", st, cString(faLastErr(c.ptr)))
	}
	return nil
}

// DeviceStatus synchronises the context's device and reports a bounded-wait expiry recorded by an attention kernel.
func (c *FAContext) DeviceStatus() error {
	if c == nil || c.ptr == 0 {
		return fmt.Errorf("FAContext.DeviceStatus: nil ctx")
	}
	if err := initFAB200(); err != nil {
		return err
	}
	if st := FAStatus(faB200.deviceStatus(c.ptr)); st != FA_OK {
		return fmt.Errorf("fa_device_status: %s (%s)", st, cString(faLastErr(c.ptr)))
	}
	return nil
}

// FANoAllocDeviceStatus is DeviceStatus for callers of FAForwardNoAlloc, which have no context.
func FANoAllocDeviceStatus() (int, error) {
	if err := initFAB200(); err != nil {
		return 0, err
	}
	rc := int(faB200.noAllocStatus())
	if rc < 0 {
		return 0, fmt.Errorf("fa_noalloc_device_status: CUDA error %d", -rc)
	}
	return rc, nil
}
