"""Host-side helpers for running the sampler on several GPUs of one node.

Two partitions, both without any framework of their own (one process per GPU,
torch.distributed only for set-up):
  * batch-parallel: rows are independent, every rank samples its own rows, no data-path
    communication (`row_partition`);
  * vocab-sharded: every rank holds a contiguous column range of every row, as a
    tensor-parallel lm_head leaves it (`shard_range`); the local pass writes one record per
    row, the records are all-gathered (NCCL inside the library) and every rank merges.
The record format of the exchange is documented by `encode_records` / `decode_records`, which
build and read records on the host (used for debugging and by the CPU tests).
"""
import numpy as np

RECORD_HDR_BYTES = 32
IDX_MASK = 0xFFFFFF


def row_partition(batch, rank, world):
    """Contiguous rows [lo, hi) of `batch` owned by `rank`."""
    lo = batch * rank // world
    hi = batch * (rank + 1) // world
    return lo, hi


def shard_range(vocab, rank, world):
    """Columns [lo, hi) of a vocab that divides evenly over `world` shards."""
    if vocab % world:
        raise ValueError("vocab must be divisible by the number of shards")
    w = vocab // world
    return rank * w, (rank + 1) * w


def record_bytes(top_k):
    return RECORD_HDR_BYTES + 8 * top_k


def float_key(z):
    """Order-preserving uint32 key of float32 values (-0 folded onto +0)."""
    b = np.ascontiguousarray(z, dtype=np.float32).view(np.uint32).copy()
    b[b == 0x80000000] = 0
    neg = (b >> 31).astype(bool)
    return np.where(neg, ~b, b | np.uint32(0x80000000)).astype(np.uint32)


def key_to_float(k):
    k = np.asarray(k, dtype=np.uint32)
    b = np.where((k >> 31).astype(bool), k ^ np.uint32(0x80000000), ~k).astype(np.uint32)
    return b.view(np.float32)


def encode_records(shard_logits, top_k, idx_offset, inv_T=1.0):
    """Records of one shard: [rows, record_bytes(top_k)] uint8.

    Header: float32 max, float32 sum of 2^((z-max)*inv_T*log2e), uint32 count, uint32 flags,
    float32 bound (a value that at least top_k tokens of the shard reach; -inf = none).
    Entries: uint64 rank keys (value key << 24 | (0xFFFFFF - global index)), best first is not
    required; unused entries are 0."""
    z = np.ascontiguousarray(shard_logits, dtype=np.float32)
    rows, vl = z.shape
    out = np.zeros((rows, record_bytes(top_k)), dtype=np.uint8)
    for r in range(rows):
        zr = z[r]
        fin = np.nonzero(zr > -np.inf)[0]
        order = fin[np.lexsort((fin, -zr[fin].astype(np.float64)))][:top_k]
        keys = (float_key(zr[order]).astype(np.uint64) << np.uint64(24)) | \
            (np.uint64(IDX_MASK) - (order.astype(np.uint64) + np.uint64(idx_offset)))
        m = zr.max() if zr.size else -np.inf
        s = np.exp2((zr.astype(np.float64) - m) * inv_T * 1.4426950408889634).sum() if np.isfinite(m) else 0.0
        hdr = out[r, :RECORD_HDR_BYTES]
        hdr[0:4] = np.array([m], dtype=np.float32).view(np.uint8)
        hdr[4:8] = np.array([s], dtype=np.float32).view(np.uint8)
        hdr[8:12] = np.array([len(order)], dtype=np.uint32).view(np.uint8)
        hdr[12:16] = np.array([1 if len(fin) > top_k else 0], dtype=np.uint32).view(np.uint8)
        hdr[16:20] = np.array([-np.inf], dtype=np.float32).view(np.uint8)
        out[r, RECORD_HDR_BYTES:RECORD_HDR_BYTES + 8 * len(order)] = keys.view(np.uint8)
    return out


def decode_records(gathered):
    """gathered: [nranks, rows, record_bytes] uint8 -> per row the candidate (values, global ids),
    the row maximum and the per-shard (max, sum) pairs."""
    g = np.ascontiguousarray(gathered, dtype=np.uint8)
    nranks, rows, rb = g.shape
    res = []
    for r in range(rows):
        vals, ids, parts = [], [], []
        for s in range(nranks):
            rec = g[s, r]
            m = rec[0:4].view(np.float32)[0]
            ssum = rec[4:8].view(np.float32)[0]
            cnt = int(rec[8:12].view(np.uint32)[0])
            keys = rec[RECORD_HDR_BYTES:RECORD_HDR_BYTES + 8 * cnt].view(np.uint64)
            alive = (keys >> np.uint64(24)) != 0
            keys = keys[alive]
            vals.append(key_to_float((keys >> np.uint64(24)).astype(np.uint32)))
            ids.append((np.uint64(IDX_MASK) - (keys & np.uint64(IDX_MASK))).astype(np.int64))
            parts.append((float(m), float(ssum)))
        res.append({"values": np.concatenate(vals), "ids": np.concatenate(ids), "parts": parts,
                    "max": max(p[0] for p in parts)})
    return res


def merged_lse(parts, inv_T=1.0):
    """Natural log-sum-exp of the whole row from the per-shard (max, sum) pairs."""
    m = max(p[0] for p in parts)
    s = sum(p[1] * np.exp2((p[0] - m) * inv_T * 1.4426950408889634) for p in parts if p[1] > 0)
    return m * inv_T + np.log(s)


class ShardedSampler:
    """A Sampler bound to one rank of a vocab-sharded group (torch.distributed for set-up only:
    rank 0's NCCL unique id is broadcast once; the data path is the library's own all-gather)."""

    def __init__(self, sampler, rank, world, dist=None):
        from .sampler import Sampler
        self.sampler, self.rank, self.world = sampler, rank, world
        uid = [Sampler.nccl_unique_id() if rank == 0 else None]
        if world > 1:
            if dist is None:
                import torch.distributed as dist
            dist.broadcast_object_list(uid, src=0)
        sampler.shard_init(uid[0], rank, world)

    def sample(self, local_logits, uniforms, top_k, temperature=1.0, top_p=0.0, **kw):
        return self.sampler.sample_sharded(local_logits, uniforms, self.rank, self.world, top_k,
                                           temperature=temperature, top_p=top_p, **kw)
