package cuda

// Multi-GPU manager for the FP8 path.  goml's Backend is single-device (deviceIdx is never set and the registry is
// keyed by device type only, backend/cuda/cuda..go:27,67; backend/backend.go:136-155).  The path shards with no
// exchange step — attention by contiguous batch*head ranges, the GEMM by 128-row tile blocks of A and C with the
// weight replicated — so the manager is one FA context and one stream per device plus three integer functions.
// Not compiled in the repository that ships this file (no Go toolchain there): the rules are the ones of
// goml_b200/multi_gpu.py (tested on CPU) and DeviceManager in goml_b200/host/goml_cuda.hpp.

import (
	"fmt"
	"runtime"
)

const GEMMTileM = 128

// ShardHeads returns the contiguous [begin, end) slice of the batch*head axis owned by rank; remainders go to the
// lowest ranks, so sizes differ by at most one head.
func ShardHeads(batchHeads, worldSize, rank int) (int, int, error) {
	if worldSize <= 0 || rank < 0 || rank >= worldSize {
		return 0, 0, fmt.Errorf("ShardHeads: bad rank %d / world size %d", rank, worldSize)
	}
	base, rem := batchHeads/worldSize, batchHeads%worldSize
	lo := rank*base + min(rank, rem)
	hi := lo + base
	if rank < rem {
		hi++
	}
	return lo, hi, nil
}

// ShardRows returns the contiguous [begin, end) block of GEMM rows owned by rank, cut on tile boundaries.
func ShardRows(M, worldSize, rank, tile int) (int, int, error) {
	if tile <= 0 {
		tile = GEMMTileM
	}
	tiles := (M + tile - 1) / tile
	tb, te, err := ShardHeads(tiles, worldSize, rank)
	if err != nil {
		return 0, 0, err
	}
	return min(tb*tile, M), min(te*tile, M), nil
}

// ShardCols is the partition for skinny-M GEMMs (fewer rows than one tile per rank): B rows / C columns are split,
// A is replicated.
func ShardCols(N, worldSize, rank int) (int, int, error) { return ShardRows(N, worldSize, rank, 256) }

// DeviceContext is the per-GPU state: device index, a stream, an FA context created with that device current.
type DeviceContext struct {
	Device int
	Stream uintptr
	FA     *FAContext
}

// DeviceManager owns one DeviceContext per GPU.  Calls for device g must be made from a goroutine that has locked its
// OS thread and made g current (WithDevice does both): the libraries use the calling thread's current device.
type DeviceManager struct {
	Devices []*DeviceContext
}

// NewDeviceManager creates a context on each of the first n devices.
func NewDeviceManager(n int) (*DeviceManager, error) {
	m := &DeviceManager{}
	for g := 0; g < n; g++ {
		var dc *DeviceContext
		err := WithDevice(g, func() error {
			stream, err := StreamCreate() // cuStreamCreate through driver.go
			if err != nil {
				return err
			}
			fa, err := FACreate()
			if err != nil {
				return err
			}
			dc = &DeviceContext{Device: g, Stream: stream, FA: fa}
			return nil
		})
		if err != nil {
			m.Close()
			return nil, fmt.Errorf("device %d: %w", g, err)
		}
		m.Devices = append(m.Devices, dc)
	}
	return m, nil
}

// WithDevice runs fn on a locked OS thread with device g current.
func WithDevice(g int, fn func() error) error {
	runtime.LockOSThread()
	defer runtime.UnlockOSThread()
	if err := SetDevice(g); err != nil { // cuCtxSetCurrent of the device's primary context (driver.go)
		return err
	}
	return fn()
}

// ForEach runs fn(rank, ctx) for every device concurrently, each on its own locked thread, and returns the first error.
func (m *DeviceManager) ForEach(fn func(rank int, dc *DeviceContext) error) error {
	errs := make(chan error, len(m.Devices))
	for r, dc := range m.Devices {
		go func(r int, dc *DeviceContext) { errs <- WithDevice(dc.Device, func() error { return fn(r, dc) }) }(r, dc)
	}
	var first error
	for range m.Devices {
		if err := <-errs; err != nil && first == nil {
			first = err
		}
	}
	return first
}

// Close destroys the FA contexts.
func (m *DeviceManager) Close() {
	for _, dc := range m.Devices {
		if dc != nil && dc.FA != nil {
			_ = WithDevice(dc.Device, func() error { dc.FA.Destroy(); return nil })
			dc.FA = nil
		}
	}
}
