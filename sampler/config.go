package sampler

// Status codes of the C ABI (include/born_sampler.h).
const (
	OK                 = 0
	ErrInvalidArgument = 1
	ErrCUDA            = 2
	ErrNoDevice        = 3
	ErrUnsupported     = 4
	ErrNCCL            = 5
	ErrDeviceTimeout   = 6
)

// Per-row status (out_status).
const (
	RowOK        = 0
	RowAllMasked = 1
	RowNaN       = 2
	RowPosInf    = 3
	RowOverflow  = 4
	RowBadToken  = 5
	RowFinished  = 6 // SampleNext: the row sampled a stop token in an earlier step
	RowBadParams = 7 // a row of a device-resident parameter array is out of range
)

const (
	MaxTopK       = 1024
	MaxCandidates = 1024
	MaxHistory    = 1024
	MaxDraft      = 16
	MaxShards     = 16

	DTypeF32  = 0
	DTypeBF16 = 1

	MemDevice = 0
	MemHost   = 1

	FlagGreedy = 1
)

// SamplingConfig holds the sampling parameters of one row.  The zero value is greedy
// decoding with every filter off, like the zero values of the reference's optimizer
// configs (internal/optim/adam.go:78-91).
type SamplingConfig struct {
	Temperature       float32 // 0 => greedy (first maximum wins)
	TopP              float32 // (0,1): nucleus over the survivors; 0 or >= 1 => off
	MinP              float32 // (0,1]: keep tokens with p >= MinP * p_max; 0 => off
	TopK              int32   // 1..MaxTopK; 0 => off
	RepetitionPenalty float32 // > 0; 1 or 0 => off
	FrequencyPenalty  float32
	PresencePenalty   float32
	Greedy            bool
}

// RowParams is born_row_params: 32 bytes, fixed-width fields, natural alignment.
type RowParams struct {
	Temperature       float32
	TopP              float32
	MinP              float32
	TopK              int32
	RepetitionPenalty float32
	FrequencyPenalty  float32
	PresencePenalty   float32
	Flags             uint32
}

func (c SamplingConfig) rowParams() RowParams {
	p := RowParams{Temperature: c.Temperature, TopP: c.TopP, MinP: c.MinP, TopK: c.TopK,
		RepetitionPenalty: c.RepetitionPenalty, FrequencyPenalty: c.FrequencyPenalty,
		PresencePenalty: c.PresencePenalty}
	if c.Greedy {
		p.Flags |= FlagGreedy
	}
	return p
}

// SampleArgs is born_sample_args, field for field.  unsafe.Pointer / uintptr fields are
// host or device addresses according to Memory.
type SampleArgs struct {
	StructSize      uint32
	Memory          uint32
	Batch           int32
	Vocab           int32
	LogitsDType     int32
	HistoryStride   int32
	LogitsRowStride int64
	Logits          uintptr
	Mask            uintptr
	MaskRowStride   int64
	History         uintptr
	HistoryLen      uintptr
	RowParams       uintptr
	Params          RowParams
	Uniforms        uintptr
	OutToken        uintptr
	OutProb         uintptr
	OutLSE          uintptr
	OutStatus       uintptr
	OutKeptIDs      uintptr
	OutKeptCount    uintptr
	KeptStride      int32
	VocabSegments   int32
}

// SpecArgs is born_spec_args.
type SpecArgs struct {
	StructSize   uint32
	Memory       uint32
	Batch        int32
	DraftLen     int32
	Vocab        int32
	TargetRows   int32
	TargetLogits uintptr
	DraftLogits  uintptr
	DraftTokens  uintptr
	UAccept      uintptr
	UResample    uintptr
	Temperature  float32
	Reserved     int32
	OutAcceptLen uintptr
	OutTokens    uintptr
	OutStatus    uintptr
}

// ShardArgs is born_shard_args.
type ShardArgs struct {
	StructSize      uint32
	Memory          uint32
	Batch           int32
	VocabLocal      int32
	LogitsDType     int32
	Rank            int32
	NRanks          int32
	TopK            int32
	LogitsRowStride int64
	Logits          uintptr
	Temperature     float32
	TopP            float32
	Uniforms        uintptr
	Packed          uintptr
	Gathered        uintptr
	OutToken        uintptr
	OutProb         uintptr
	OutLSE          uintptr
	OutStatus       uintptr
}
