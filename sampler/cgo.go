//go:build cgo

package sampler

/*
#cgo CFLAGS: -I${SRCDIR}/../include
#cgo LDFLAGS: -L${SRCDIR}/../born_b200 -lborn_sampler -Wl,-rpath,${SRCDIR}/../born_b200
#include "born_sampler.h"
*/
import "C"

import "unsafe"

// The Go structs of config.go mirror the C structs field for field (fixed-width fields,
// natural alignment); struct_size guards against drift.
type cgoBinding struct{}

func load() (binding, error) { return cgoBinding{}, nil }

func h2p(h uintptr) unsafe.Pointer { return unsafe.Pointer(h) } //nolint:govet // opaque C handle

func (cgoBinding) create(device, maxBatch, maxVocab, maxK int32) (uintptr, int32) {
	var h unsafe.Pointer
	rc := C.born_sampler_create(C.int32_t(device), C.int32_t(maxBatch), C.int32_t(maxVocab), C.int32_t(maxK), &h)
	return uintptr(h), int32(rc)
}
func (cgoBinding) destroy(h uintptr) { C.born_sampler_destroy(h2p(h)) }
func (cgoBinding) sample(h uintptr, a *SampleArgs, st uintptr) int32 {
	return int32(C.born_sample(h2p(h), (*C.born_sample_args)(unsafe.Pointer(a)), h2p(st)))
}
func (cgoBinding) sampleStatic(a *SampleArgs, st uintptr) int32 {
	return int32(C.born_sample_static((*C.born_sample_args)(unsafe.Pointer(a)), h2p(st)))
}
func (cgoBinding) reserve(h uintptr, a *SampleArgs) int32 {
	return int32(C.born_sampler_reserve(h2p(h), (*C.born_sample_args)(unsafe.Pointer(a))))
}
func (cgoBinding) checkError(h uintptr) int32   { return int32(C.born_check_error(h2p(h))) }
func (cgoBinding) fallbackRows(h uintptr) int64 { return int64(C.born_fallback_rows(h2p(h))) }
func (cgoBinding) specVerify(h uintptr, a *SpecArgs, st uintptr) int32 {
	return int32(C.born_spec_verify(h2p(h), (*C.born_spec_args)(unsafe.Pointer(a)), h2p(st)))
}
func (cgoBinding) shardRecordBytes(k int32) int32 { return int32(C.born_shard_record_bytes(C.int32_t(k))) }
func (cgoBinding) shardUniqueID(out *[128]byte) int32 {
	return int32(C.born_shard_unique_id(unsafe.Pointer(out)))
}
func (cgoBinding) shardInit(h uintptr, id *[128]byte, rank, nranks int32) int32 {
	return int32(C.born_shard_init(h2p(h), unsafe.Pointer(id), C.int32_t(rank), C.int32_t(nranks)))
}
func (cgoBinding) shardLocal(h uintptr, a *ShardArgs, st uintptr) int32 {
	return int32(C.born_shard_local(h2p(h), (*C.born_shard_args)(unsafe.Pointer(a)), h2p(st)))
}
func (cgoBinding) shardMerge(h uintptr, a *ShardArgs, st uintptr) int32 {
	return int32(C.born_shard_merge(h2p(h), (*C.born_shard_args)(unsafe.Pointer(a)), h2p(st)))
}
func (cgoBinding) sampleSharded(h uintptr, a *ShardArgs, st uintptr) int32 {
	return int32(C.born_sample_sharded(h2p(h), (*C.born_shard_args)(unsafe.Pointer(a)), h2p(st)))
}
func (cgoBinding) historyCreate(h uintptr, capacity int32) int32 {
	return int32(C.born_history_create(h2p(h), C.int32_t(capacity)))
}
func (cgoBinding) historyReset(h uintptr, tokens, lens uintptr, batch, stride int32, memory uint32, st uintptr) int32 {
	return int32(C.born_history_reset(h2p(h), (*C.int32_t)(h2p(tokens)), (*C.int32_t)(h2p(lens)), C.int32_t(batch),
		C.int32_t(stride), C.uint32_t(memory), h2p(st)))
}
func (cgoBinding) historySetStopTokens(h uintptr, ids *int32, n int32) int32 {
	return int32(C.born_history_set_stop_tokens(h2p(h), (*C.int32_t)(unsafe.Pointer(ids)), C.int32_t(n)))
}
func (cgoBinding) historyRead(h uintptr, tokens, total, finished uintptr, batch int32, memory uint32, st uintptr) int32 {
	return int32(C.born_history_read(h2p(h), (*C.int32_t)(h2p(tokens)), (*C.int32_t)(h2p(total)), (*C.int32_t)(h2p(finished)),
		C.int32_t(batch), C.uint32_t(memory), h2p(st)))
}
func (cgoBinding) sampleNext(h uintptr, a *SampleArgs, st uintptr) int32 {
	return int32(C.born_sample_next(h2p(h), (*C.born_sample_args)(unsafe.Pointer(a)), h2p(st)))
}
func (cgoBinding) maskBegin(h uintptr, batch, wordsPerRow int32, host *uintptr) int32 {
	return int32(C.born_mask_begin(h2p(h), C.int32_t(batch), C.int32_t(wordsPerRow), (**C.uint32_t)(unsafe.Pointer(host))))
}
func (cgoBinding) maskCommit(h uintptr, device *uintptr) int32 {
	return int32(C.born_mask_commit(h2p(h), (**C.uint32_t)(unsafe.Pointer(device))))
}
func (cgoBinding) maskWait(h uintptr, st uintptr) int32 { return int32(C.born_mask_wait(h2p(h), h2p(st))) }
func (cgoBinding) lastError(h uintptr) string { return C.GoString(C.born_last_error(h2p(h))) }
func (cgoBinding) version() string            { return C.GoString(C.born_version()) }
