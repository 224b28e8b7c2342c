package sampler

import "fmt"

// Error is a runtime failure reported by the library (CUDA, NCCL, device timeout,
// unsupported request, no device).  Programmer errors (ErrInvalidArgument) never reach the
// caller as Error: the wrappers panic, as the reference's backends do.
type Error struct {
	Code    int32
	Message string
}

func (e *Error) Error() string { return fmt.Sprintf("born sampler: error %d: %s", e.Code, e.Message) }

// RowError reports the first row whose status is not RowOK; that row's token is -1.
type RowError struct {
	Row    int
	Status int32
}

func (e *RowError) Error() string {
	names := map[int32]string{RowAllMasked: "every token masked", RowNaN: "NaN logit", RowPosInf: "+inf logit",
		RowOverflow: "shard record not exact", RowBadToken: "draft token out of range",
		RowFinished: "row finished at a stop token", RowBadParams: "sampling parameters out of range"}
	if e.Status == 100+ErrDeviceTimeout {
		return fmt.Sprintf("born sampler: row %d: a bounded on-device wait gave up", e.Row)
	}
	return fmt.Sprintf("born sampler: row %d: %s", e.Row, names[e.Status])
}

func check(code int32, msg func() string) error {
	switch code {
	case OK:
		return nil
	case ErrInvalidArgument:
		panic("born sampler: " + msg())
	default:
		return &Error{Code: code, Message: msg()}
	}
}

func firstBadRow(status []int32) error {
	for b, st := range status {
		if st != RowOK {
			return &RowError{Row: b, Status: st}
		}
	}
	return nil
}
