package sampler

// uncompiled: no Go toolchain in the build environment of this file; it is written against
// include/born_sampler.h and the loaders of cgo.go / purego.go.

import (
	"runtime"
	"unsafe"
)

// The generate loop around the sampler.  The reference's call site of this path is a host loop
// that takes the arg-max of each batch's output (examples/mnist/main.go:229-245); a language
// model does the same once per token and feeds the token back.  These methods keep the loop's
// state -- token history, stop flags, the next grammar mask -- on the device.

// HistoryCreate allocates the device-resident history: the last `capacity` tokens per row.
func (s *CUDASampler) HistoryCreate(capacity int) error {
	return check(s.b.historyCreate(s.h, int32(capacity)), s.msg)
}

// HistoryReset loads prompts (host memory, [batch, stride], lens may be nil) and clears the
// finished flags.
func (s *CUDASampler) HistoryReset(tokens []int32, lens []int32, batch, stride int) error {
	var pin runtime.Pinner
	defer pin.Unpin()
	var tp, lp uintptr
	if len(tokens) > 0 {
		pin.Pin(&tokens[0])
		tp = uintptr(unsafe.Pointer(&tokens[0]))
	}
	if len(lens) > 0 {
		pin.Pin(&lens[0])
		lp = uintptr(unsafe.Pointer(&lens[0]))
	}
	return check(s.b.historyReset(s.h, tp, lp, int32(batch), int32(stride), MemHost, 0), s.msg)
}

// SetStopTokens takes up to 8 ids; a row that samples one is finished from the next step on.
func (s *CUDASampler) SetStopTokens(ids []int32) error {
	var p *int32
	if len(ids) > 0 {
		p = &ids[0]
	}
	return check(s.b.historySetStopTokens(s.h, p, int32(len(ids))), s.msg)
}

// HistoryRead copies the state to the host: tokens [batch, capacity] in ring order, tokens
// appended since the reset, finished flags.
func (s *CUDASampler) HistoryRead(batch, capacity int) (tokens, total, finished []int32, err error) {
	tokens = make([]int32, batch*capacity)
	total = make([]int32, batch)
	finished = make([]int32, batch)
	var pin runtime.Pinner
	defer pin.Unpin()
	pin.Pin(&tokens[0])
	pin.Pin(&total[0])
	pin.Pin(&finished[0])
	err = check(s.b.historyRead(s.h, uintptr(unsafe.Pointer(&tokens[0])), uintptr(unsafe.Pointer(&total[0])),
		uintptr(unsafe.Pointer(&finished[0])), int32(batch), MemHost, 0), s.msg)
	return tokens, total, finished, err
}

// SampleNext is SampleDevice over the device-resident history: a.History must be 0; the
// kernel appends every row's token before it exits.
func (s *CUDASampler) SampleNext(a *SampleArgs, stream uintptr) error {
	a.StructSize = uint32(unsafe.Sizeof(*a))
	a.Memory = MemDevice
	return check(s.b.sampleNext(s.h, a, stream), s.msg)
}

// MaskBegin returns the pinned host buffer ([batch, wordsPerRow] words) to fill with the next
// step's grammar mask while the previous step's kernel runs.
func (s *CUDASampler) MaskBegin(batch, wordsPerRow int) ([]uint32, error) {
	var host uintptr
	if err := check(s.b.maskBegin(s.h, int32(batch), int32(wordsPerRow), &host), s.msg); err != nil {
		return nil, err
	}
	return unsafe.Slice((*uint32)(unsafe.Pointer(host)), batch*wordsPerRow), nil //nolint:govet // pinned C memory
}

// MaskCommit starts the copy to the device and returns the device pointer for a.Mask.
func (s *CUDASampler) MaskCommit() (uintptr, error) {
	var dev uintptr
	err := check(s.b.maskCommit(s.h, &dev), s.msg)
	return dev, err
}

// MaskWait makes `stream` wait for the committed mask.
func (s *CUDASampler) MaskWait(stream uintptr) error { return check(s.b.maskWait(s.h, stream), s.msg) }
