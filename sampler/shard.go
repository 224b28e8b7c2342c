package sampler

import "unsafe"

// The vocab-sharded path (a tensor-parallel lm_head: every rank holds a contiguous column
// range of every row).  One process per GPU; rank 0 makes the NCCL unique id, the 128 bytes
// travel over whatever channel the host already has, every rank calls ShardInit.  All
// pointers are device memory.

// ShardUniqueID returns the 128-byte NCCL unique id (call on rank 0).
func ShardUniqueID() ([128]byte, error) {
	var id [128]byte
	b, err := load()
	if err != nil {
		return id, err
	}
	return id, check(b.shardUniqueID(&id), func() string { return b.lastError(0) })
}

func (s *CUDASampler) ShardInit(id [128]byte, rank, nranks int) error {
	return check(s.b.shardInit(s.h, &id, int32(rank), int32(nranks)), s.msg)
}

// ShardRecordBytes is the size of one packed record: 32 + 8 * topK.
func (s *CUDASampler) ShardRecordBytes(topK int) int { return int(s.b.shardRecordBytes(int32(topK))) }

func prepShard(a *ShardArgs) {
	a.StructSize = uint32(unsafe.Sizeof(*a))
	a.Memory = MemDevice
}

// ShardLocal writes one packed record per row (the shard's k best tokens with global ids,
// its maximum, its share of the log-sum-exp) into a.Packed.
func (s *CUDASampler) ShardLocal(a *ShardArgs, stream uintptr) error {
	prepShard(a)
	return check(s.b.shardLocal(s.h, a, stream), s.msg)
}

// ShardMerge draws the tokens from the all-gathered records [nranks, batch, record].
func (s *CUDASampler) ShardMerge(a *ShardArgs, stream uintptr) error {
	prepShard(a)
	return check(s.b.shardMerge(s.h, a, stream), s.msg)
}

// SampleSharded = ShardLocal, one ncclAllGather inside the library, ShardMerge.
func (s *CUDASampler) SampleSharded(a *ShardArgs, stream uintptr) error {
	prepShard(a)
	return check(s.b.sampleSharded(s.h, a, stream), s.msg)
}
