package sampler

import (
	"runtime"
	"unsafe"
)

// binding is what both loaders (cgo.go, purego.go) provide: the entry points of
// include/born_sampler.h with Go-friendly scalar types.
type binding interface {
	create(device, maxBatch, maxVocab, maxK int32) (handle uintptr, code int32)
	destroy(handle uintptr)
	sample(handle uintptr, a *SampleArgs, stream uintptr) int32
	sampleStatic(a *SampleArgs, stream uintptr) int32
	reserve(handle uintptr, a *SampleArgs) int32
	checkError(handle uintptr) int32
	fallbackRows(handle uintptr) int64
	specVerify(handle uintptr, a *SpecArgs, stream uintptr) int32
	shardRecordBytes(topK int32) int32
	shardUniqueID(out *[128]byte) int32
	shardInit(handle uintptr, id *[128]byte, rank, nranks int32) int32
	shardLocal(handle uintptr, a *ShardArgs, stream uintptr) int32
	shardMerge(handle uintptr, a *ShardArgs, stream uintptr) int32
	sampleSharded(handle uintptr, a *ShardArgs, stream uintptr) int32
	historyCreate(handle uintptr, capacity int32) int32
	historyReset(handle uintptr, tokens, lens uintptr, batch, stride int32, memory uint32, stream uintptr) int32
	historySetStopTokens(handle uintptr, ids *int32, n int32) int32
	historyRead(handle uintptr, tokens, total, finished uintptr, batch int32, memory uint32, stream uintptr) int32
	sampleNext(handle uintptr, a *SampleArgs, stream uintptr) int32
	maskBegin(handle uintptr, batch, wordsPerRow int32, host *uintptr) int32
	maskCommit(handle uintptr, device *uintptr) int32
	maskWait(handle uintptr, stream uintptr) int32
	lastError(handle uintptr) string
	version() string
}

// SamplerBackend is the capability a backend offers when it can sample tokens from
// logits.  It is discovered the way the reference discovers ReLUBackend
// (internal/nn/activation.go:41-52):
//
//	if sb, ok := any(backend).(sampler.SamplerBackend); ok { tokens, err = sb.Sample(...) }
type SamplerBackend interface {
	// Sample draws one token per row of logits [batch, vocab] (row-major float32, host
	// memory: the layout of tensor.RawTensor.AsFloat32, internal/tensor/raw.go:145-160).
	Sample(logits []float32, batch, vocab int, cfg SamplingConfig, st *State) (tokens []int32, probs []float32, err error)
}

// State is what a decode loop carries between steps: the token history of every row (for
// the repetition / frequency / presence penalties) and the uniform variates of the step.
type State struct {
	History       []int32 // [batch, HistoryStride] prior token ids; nil => no penalties
	HistoryStride int
	HistoryLen    []int32   // valid ids per row; nil => HistoryStride
	Mask          []uint32  // [batch, ceil(vocab/32)] grammar bitset; nil => none
	Uniforms      []float32 // [batch] in [0,1); may be nil when every row is greedy
}

// CUDASampler owns one handle of the library (one device workspace, one stream of calls;
// not safe for concurrent use -- distinct samplers are independent).
type CUDASampler struct {
	b binding
	h uintptr
}

// New creates a sampler on `device` for up to maxBatch rows of maxVocab tokens.  There is
// no CPU fallback: without a usable sm_100 device the error is ErrNoDevice.
func New(device, maxBatch, maxVocab int) (*CUDASampler, error) {
	b, err := load()
	if err != nil {
		return nil, err
	}
	h, code := b.create(int32(device), int32(maxBatch), int32(maxVocab), MaxTopK)
	if err := check(code, func() string { return b.lastError(0) }); err != nil {
		return nil, err
	}
	s := &CUDASampler{b: b, h: h}
	runtime.SetFinalizer(s, func(s *CUDASampler) { s.Close() })
	return s, nil
}

func (s *CUDASampler) Close() {
	if s.h != 0 {
		s.b.destroy(s.h)
		s.h = 0
	}
}

func (s *CUDASampler) Version() string { return s.b.version() }

func (s *CUDASampler) msg() string { return s.b.lastError(s.h) }

// Sample implements SamplerBackend over host memory (BORN_MEM_HOST: the call copies in,
// runs, copies out and returns after the stream has drained).
func (s *CUDASampler) Sample(logits []float32, batch, vocab int, cfg SamplingConfig, st *State) ([]int32, []float32, error) {
	if len(logits) != batch*vocab {
		panic("sampler: logits must be [batch, vocab]")
	}
	tokens := make([]int32, batch)
	probs := make([]float32, batch)
	status := make([]int32, batch)
	var a SampleArgs
	a.StructSize = uint32(unsafe.Sizeof(a))
	a.Memory = MemHost
	a.Batch, a.Vocab = int32(batch), int32(vocab)
	a.LogitsDType = DTypeF32
	a.LogitsRowStride = int64(vocab)
	a.Params = cfg.rowParams()
	var pin runtime.Pinner // the args struct holds Go pointers: pinned for the duration of the call
	defer pin.Unpin()
	ptr := func(p unsafe.Pointer) uintptr { pin.Pin(p); return uintptr(p) }
	a.Logits = ptr(unsafe.Pointer(&logits[0]))
	if st != nil {
		if len(st.History) > 0 {
			a.History = ptr(unsafe.Pointer(&st.History[0]))
			a.HistoryStride = int32(st.HistoryStride)
			if len(st.HistoryLen) > 0 {
				a.HistoryLen = ptr(unsafe.Pointer(&st.HistoryLen[0]))
			}
		}
		if len(st.Mask) > 0 {
			a.Mask = ptr(unsafe.Pointer(&st.Mask[0]))
			a.MaskRowStride = int64((vocab + 31) / 32)
		}
		if len(st.Uniforms) > 0 {
			a.Uniforms = ptr(unsafe.Pointer(&st.Uniforms[0]))
		}
	}
	a.OutToken = ptr(unsafe.Pointer(&tokens[0]))
	a.OutProb = ptr(unsafe.Pointer(&probs[0]))
	a.OutStatus = ptr(unsafe.Pointer(&status[0]))
	if err := check(s.b.sample(s.h, &a, 0), s.msg); err != nil {
		return nil, nil, err
	}
	return tokens, probs, firstBadRow(status)
}

// SampleDevice is the asynchronous form: every pointer in `a` is device memory, the call
// returns as soon as the kernels are queued on `stream` (a cudaStream_t, 0 = default).
// Bounded-wait expiries of such calls are read with CheckError.
func (s *CUDASampler) SampleDevice(a *SampleArgs, stream uintptr) error {
	a.StructSize = uint32(unsafe.Sizeof(*a))
	a.Memory = MemDevice
	return check(s.b.sample(s.h, a, stream), s.msg)
}

// Reserve allocates now whatever scratch a later call with these arguments would allocate
// on first use.
func (s *CUDASampler) Reserve(a *SampleArgs) error {
	a.StructSize = uint32(unsafe.Sizeof(*a))
	return check(s.b.reserve(s.h, a), s.msg)
}

// CheckError reads and clears the device error word (synchronises the device).
func (s *CUDASampler) CheckError() error { return check(s.b.checkError(s.h), s.msg) }

// FallbackRows returns how many rows took the exact multi-pass search since the last call.
func (s *CUDASampler) FallbackRows() int64 { return s.b.fallbackRows(s.h) }

// SampleStatic is the allocation-free entry point (born_sample_static): no handle, scratch
// in a fixed array inside the library image; device pointers only, at most 256 rows per
// call, one call at a time per GPU, first call before any stream capture.
func SampleStatic(a *SampleArgs, stream uintptr) error {
	b, err := load()
	if err != nil {
		return err
	}
	a.StructSize = uint32(unsafe.Sizeof(*a))
	a.Memory = MemDevice
	return check(b.sampleStatic(a, stream), func() string { return b.lastError(0) })
}
