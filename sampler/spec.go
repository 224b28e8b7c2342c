package sampler

import (
	"runtime"
	"unsafe"
)

// SpecResult is the outcome of speculative-decoding verification for one batch.
type SpecResult struct {
	AcceptLen []int32 // [batch] accepted draft tokens
	Tokens    []int32 // [batch, K+1] accepted tokens, then the resampled / bonus token, -1 padded
}

// SpecVerify accepts or rejects K draft tokens per sequence against the target logits
// (host memory, float32): accept x_j iff u * q_j(x_j) < p_j(x_j); at the first rejection a
// token is drawn from max(0, p_j - q_j); when all are accepted and target has K+1 rows the
// bonus token is drawn from the last one.
func (s *CUDASampler) SpecVerify(target, draft []float32, draftTokens []int32, uAccept, uResample []float32,
	batch, draftLen, vocab, targetRows int, temperature float32) (*SpecResult, error) {
	if len(target) != batch*targetRows*vocab || len(draft) != batch*draftLen*vocab ||
		len(draftTokens) != batch*draftLen || len(uAccept) != batch*draftLen || len(uResample) != batch*(draftLen+1) {
		panic("sampler: SpecVerify: slice lengths do not match the shapes")
	}
	res := &SpecResult{AcceptLen: make([]int32, batch), Tokens: make([]int32, batch*(draftLen+1))}
	status := make([]int32, batch)
	var a SpecArgs
	a.StructSize = uint32(unsafe.Sizeof(a))
	a.Memory = MemHost
	a.Batch, a.DraftLen, a.Vocab, a.TargetRows = int32(batch), int32(draftLen), int32(vocab), int32(targetRows)
	a.Temperature = temperature
	var pin runtime.Pinner
	defer pin.Unpin()
	ptr := func(p unsafe.Pointer) uintptr { pin.Pin(p); return uintptr(p) }
	a.TargetLogits = ptr(unsafe.Pointer(&target[0]))
	a.DraftLogits = ptr(unsafe.Pointer(&draft[0]))
	a.DraftTokens = ptr(unsafe.Pointer(&draftTokens[0]))
	a.UAccept = ptr(unsafe.Pointer(&uAccept[0]))
	a.UResample = ptr(unsafe.Pointer(&uResample[0]))
	a.OutAcceptLen = ptr(unsafe.Pointer(&res.AcceptLen[0]))
	a.OutTokens = ptr(unsafe.Pointer(&res.Tokens[0]))
	a.OutStatus = ptr(unsafe.Pointer(&status[0]))
	if err := check(s.b.specVerify(s.h, &a, 0), s.msg); err != nil {
		return nil, err
	}
	return res, firstBadRow(status)
}
