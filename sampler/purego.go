//go:build !cgo

package sampler

// No-cgo loader: dlopen + register-based trampolines (github.com/ebitengine/purego).  Every
// entry point of the library takes at most five scalar / pointer arguments and no struct by
// value, so plain function-pointer registration is enough.

import (
	"fmt"
	"os"
	"sync"
	"unsafe"

	"github.com/ebitengine/purego"
)

type puregoBinding struct {
	fCreate        func(device, maxBatch, maxVocab, maxK int32, out *uintptr) int32
	fDestroy       func(h uintptr) int32
	fSample        func(h uintptr, a *SampleArgs, stream uintptr) int32
	fSampleStatic  func(a *SampleArgs, stream uintptr) int32
	fReserve       func(h uintptr, a *SampleArgs) int32
	fCheckError    func(h uintptr) int32
	fFallbackRows  func(h uintptr) int64
	fSpecVerify    func(h uintptr, a *SpecArgs, stream uintptr) int32
	fRecordBytes   func(k int32) int32
	fUniqueID      func(out *[128]byte) int32
	fShardInit     func(h uintptr, id *[128]byte, rank, nranks int32) int32
	fShardLocal    func(h uintptr, a *ShardArgs, stream uintptr) int32
	fShardMerge    func(h uintptr, a *ShardArgs, stream uintptr) int32
	fSampleSharded func(h uintptr, a *ShardArgs, stream uintptr) int32
	fHistCreate    func(h uintptr, capacity int32) int32
	fHistReset     func(h uintptr, tokens, lens uintptr, batch, stride int32, memory uint32, stream uintptr) int32
	fHistStop      func(h uintptr, ids *int32, n int32) int32
	fHistRead      func(h uintptr, tokens, total, finished uintptr, batch int32, memory uint32, stream uintptr) int32
	fSampleNext    func(h uintptr, a *SampleArgs, stream uintptr) int32
	fMaskBegin     func(h uintptr, batch, words int32, host *uintptr) int32
	fMaskCommit    func(h uintptr, device *uintptr) int32
	fMaskWait      func(h uintptr, stream uintptr) int32
	fLastError     func(h uintptr) *byte
	fVersion       func() *byte
}

var (
	once    sync.Once
	loaded  *puregoBinding
	loadErr error
)

func load() (binding, error) {
	once.Do(func() {
		path := os.Getenv("BORN_SAMPLER_LIB")
		if path == "" {
			path = "libborn_sampler.so"
		}
		lib, err := purego.Dlopen(path, purego.RTLD_NOW|purego.RTLD_GLOBAL)
		if err != nil {
			loadErr = fmt.Errorf("born sampler: cannot load %s (there is no CPU fallback): %w", path, err)
			return
		}
		b := &puregoBinding{}
		purego.RegisterLibFunc(&b.fCreate, lib, "born_sampler_create")
		purego.RegisterLibFunc(&b.fDestroy, lib, "born_sampler_destroy")
		purego.RegisterLibFunc(&b.fSample, lib, "born_sample")
		purego.RegisterLibFunc(&b.fSampleStatic, lib, "born_sample_static")
		purego.RegisterLibFunc(&b.fReserve, lib, "born_sampler_reserve")
		purego.RegisterLibFunc(&b.fCheckError, lib, "born_check_error")
		purego.RegisterLibFunc(&b.fFallbackRows, lib, "born_fallback_rows")
		purego.RegisterLibFunc(&b.fSpecVerify, lib, "born_spec_verify")
		purego.RegisterLibFunc(&b.fRecordBytes, lib, "born_shard_record_bytes")
		purego.RegisterLibFunc(&b.fUniqueID, lib, "born_shard_unique_id")
		purego.RegisterLibFunc(&b.fShardInit, lib, "born_shard_init")
		purego.RegisterLibFunc(&b.fShardLocal, lib, "born_shard_local")
		purego.RegisterLibFunc(&b.fShardMerge, lib, "born_shard_merge")
		purego.RegisterLibFunc(&b.fSampleSharded, lib, "born_sample_sharded")
		purego.RegisterLibFunc(&b.fHistCreate, lib, "born_history_create")
		purego.RegisterLibFunc(&b.fHistReset, lib, "born_history_reset")
		purego.RegisterLibFunc(&b.fHistStop, lib, "born_history_set_stop_tokens")
		purego.RegisterLibFunc(&b.fHistRead, lib, "born_history_read")
		purego.RegisterLibFunc(&b.fSampleNext, lib, "born_sample_next")
		purego.RegisterLibFunc(&b.fMaskBegin, lib, "born_mask_begin")
		purego.RegisterLibFunc(&b.fMaskCommit, lib, "born_mask_commit")
		purego.RegisterLibFunc(&b.fMaskWait, lib, "born_mask_wait")
		purego.RegisterLibFunc(&b.fLastError, lib, "born_last_error")
		purego.RegisterLibFunc(&b.fVersion, lib, "born_version")
		loaded = b
	})
	if loadErr != nil {
		return nil, loadErr
	}
	return loaded, nil
}

func cstr(p *byte) string {
	if p == nil {
		return ""
	}
	n := 0
	for *(*byte)(unsafe.Add(unsafe.Pointer(p), n)) != 0 {
		n++
	}
	return string(unsafe.Slice(p, n))
}

func (b *puregoBinding) create(device, maxBatch, maxVocab, maxK int32) (uintptr, int32) {
	var h uintptr
	rc := b.fCreate(device, maxBatch, maxVocab, maxK, &h)
	return h, rc
}
func (b *puregoBinding) destroy(h uintptr)                                     { b.fDestroy(h) }
func (b *puregoBinding) sample(h uintptr, a *SampleArgs, st uintptr) int32     { return b.fSample(h, a, st) }
func (b *puregoBinding) sampleStatic(a *SampleArgs, st uintptr) int32          { return b.fSampleStatic(a, st) }
func (b *puregoBinding) reserve(h uintptr, a *SampleArgs) int32                { return b.fReserve(h, a) }
func (b *puregoBinding) checkError(h uintptr) int32                            { return b.fCheckError(h) }
func (b *puregoBinding) fallbackRows(h uintptr) int64                          { return b.fFallbackRows(h) }
func (b *puregoBinding) specVerify(h uintptr, a *SpecArgs, st uintptr) int32   { return b.fSpecVerify(h, a, st) }
func (b *puregoBinding) shardRecordBytes(k int32) int32                        { return b.fRecordBytes(k) }
func (b *puregoBinding) shardUniqueID(out *[128]byte) int32                    { return b.fUniqueID(out) }
func (b *puregoBinding) shardLocal(h uintptr, a *ShardArgs, st uintptr) int32  { return b.fShardLocal(h, a, st) }
func (b *puregoBinding) shardMerge(h uintptr, a *ShardArgs, st uintptr) int32  { return b.fShardMerge(h, a, st) }
func (b *puregoBinding) lastError(h uintptr) string                            { return cstr(b.fLastError(h)) }
func (b *puregoBinding) version() string                                       { return cstr(b.fVersion()) }
func (b *puregoBinding) shardInit(h uintptr, id *[128]byte, rank, nranks int32) int32 {
	return b.fShardInit(h, id, rank, nranks)
}
func (b *puregoBinding) sampleSharded(h uintptr, a *ShardArgs, st uintptr) int32 {
	return b.fSampleSharded(h, a, st)
}
func (b *puregoBinding) historyCreate(h uintptr, capacity int32) int32 { return b.fHistCreate(h, capacity) }
func (b *puregoBinding) historyReset(h uintptr, tokens, lens uintptr, batch, stride int32, memory uint32, st uintptr) int32 {
	return b.fHistReset(h, tokens, lens, batch, stride, memory, st)
}
func (b *puregoBinding) historySetStopTokens(h uintptr, ids *int32, n int32) int32 { return b.fHistStop(h, ids, n) }
func (b *puregoBinding) historyRead(h uintptr, tokens, total, finished uintptr, batch int32, memory uint32, st uintptr) int32 {
	return b.fHistRead(h, tokens, total, finished, batch, memory, st)
}
func (b *puregoBinding) sampleNext(h uintptr, a *SampleArgs, st uintptr) int32 { return b.fSampleNext(h, a, st) }
func (b *puregoBinding) maskBegin(h uintptr, batch, words int32, host *uintptr) int32 {
	return b.fMaskBegin(h, batch, words, host)
}
func (b *puregoBinding) maskCommit(h uintptr, device *uintptr) int32 { return b.fMaskCommit(h, device) }
func (b *puregoBinding) maskWait(h uintptr, st uintptr) int32        { return b.fMaskWait(h, st) }
