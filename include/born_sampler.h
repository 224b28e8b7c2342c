/*
 * born_sampler.h -- C ABI of libborn_sampler.so: token sampling and constrained decoding
 * over row-major [batch, vocab] logits on NVIDIA B200 (sm_100a).
 *
 * The library is what a Go host (born) binds through cgo or a purego-style dlopen: every
 * entry point takes at most a handle, one pointer to a flat fixed-width struct and a
 * stream, and returns an int32 status (0 = BORN_OK).  No struct is passed by value, no
 * varargs, no C++ types.
 *
 * Where each entry point sits relative to the reference (born v0.1.1, paths inside that
 * project):
 *   - logits layout: contiguous row-major [batch, vocab], row b at b*vocab, int32 token
 *     indices -- internal/tensor/shape.go:52-63, internal/nn/cross_entropy.go:73,85.
 *   - the call replaces the per-row consumers of logits that the reference has:
 *     nn.Accuracy / argmax (internal/nn/cross_entropy.go:241-284, greedy decode) and the
 *     max-shifted softmax / log-sum-exp (internal/autodiff/ops/softmax.go:214-238,
 *     internal/nn/cross_entropy.go:126-153).
 *   - the reference's backend idiom is "extra capabilities are extra methods found by type
 *     assertion" (internal/nn/activation.go:7-20,41-52) on top of tensor.Backend
 *     (internal/tensor/backend.go:12-33); the host-side wrapper exposes these entry points
 *     as such a capability (SamplerBackend).  Programmer errors panic on the Go side
 *     (internal/backend/cpu/backend.go:35-37), runtime failures are returned as errors
 *     (internal/tensor/raw.go:89-92): BORN_ERR_INVALID_ARGUMENT maps to the former, the
 *     CUDA/NCCL codes to the latter.
 *
 * Ownership: the caller owns every input and output buffer.  The library owns only its
 * workspace.  What the sampling kernel needs (segment records, mass blocks, tickets) is
 * allocated in born_sampler_create and never per call.  Three kinds of scratch are grown to
 * the largest request seen instead, because their size depends on the call: the staging
 * mirrors of BORN_MEM_HOST calls, the aligned fp32 copy that whole-vocabulary rows need when
 * their logits are not 16-byte aligned or are bf16 with history penalties, and the scratch of
 * born_spec_verify.  born_sampler_reserve makes such a request ahead of time, so that no
 * later call of that shape allocates; born_shard_init sizes the exchange buffers.
 * Threading: one handle = one stream of calls; distinct handles are independent.
 */
#ifndef BORN_SAMPLER_H
#define BORN_SAMPLER_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes (return values) ---- */
#define BORN_OK 0
#define BORN_ERR_INVALID_ARGUMENT 1 /* null pointer, bad size, parameter out of range */
#define BORN_ERR_CUDA 2             /* a CUDA runtime call failed; see born_last_error */
#define BORN_ERR_NO_DEVICE 3        /* no usable CUDA device (the library has no CPU path) */
#define BORN_ERR_UNSUPPORTED 4      /* valid request outside the limits below */
#define BORN_ERR_NCCL 5             /* NCCL missing or a collective failed */
#define BORN_ERR_DEVICE_TIMEOUT 6   /* a bounded on-device wait gave up; outputs are invalid */

/* ---- per-row status (out_status[b]) ---- */
#define BORN_ROW_OK 0
#define BORN_ROW_ALL_MASKED 1 /* no allowed token with a logit above -inf: token = -1 */
#define BORN_ROW_NAN 2        /* NaN logit among the allowed tokens: token = -1 */
#define BORN_ROW_POS_INF 3    /* +inf logit among the allowed tokens: token = -1 */
#define BORN_ROW_OVERFLOW 4   /* only from the vocab-sharded path: a shard record could not be made exact */
#define BORN_ROW_BAD_TOKEN 5  /* speculative verify: draft token outside [0, vocab) */
#define BORN_ROW_BAD_PARAMS 7 /* a row of a device-resident row_params array is out of range: token = -1 */
#define BORN_ROW_FINISHED 6   /* born_sample_next: the row sampled a stop token in an earlier step; token = -1 */

/* ---- limits ---- */
#define BORN_MAX_TOP_K 1024
#define BORN_MAX_CANDIDATES 1024   /* top_k * shards in the sharded path; longest kept-id list */
#define BORN_MAX_HISTORY 1024      /* history ids per row */
#define BORN_MAX_VOCAB ((1 << 24) - 4096)
#define BORN_MAX_DRAFT 16          /* speculative draft length */
#define BORN_MAX_SHARDS 16

#define BORN_DTYPE_F32 0
#define BORN_DTYPE_BF16 1

#define BORN_MEM_DEVICE 0 /* every pointer in the args struct is device memory */
#define BORN_MEM_HOST 1   /* every pointer is host memory; the call copies in, runs, copies
                             out and returns after the stream has drained */

#define BORN_FLAG_GREEDY 1u
#define BORN_FLAG_FULL_VOCAB 2u /* accepted and ignored: every parameter set is exact over the whole vocabulary */

/* Sampling parameters of one row (32 bytes).  Zero means "off" for every filter, as in
 * the reference's config structs (internal/optim/adam.go:78-91). */
typedef struct born_row_params {
    float temperature;        /* 0 => greedy (first maximum wins) */
    float top_p;              /* (0,1): nucleus over the survivors; 0 or >= 1 => off */
    float min_p;              /* (0,1]: keep tokens with p >= min_p * p_max; 0 => off */
    int32_t top_k;            /* 1..BORN_MAX_TOP_K; 0 => off */
    float repetition_penalty; /* > 0; 1 or 0 => off; z>0 ? z/r : z*r once per distinct token */
    float frequency_penalty;  /* z -= f * count */
    float presence_penalty;   /* z -= p once per distinct token */
    uint32_t flags;           /* BORN_FLAG_GREEDY, BORN_FLAG_FULL_VOCAB */
} born_row_params;

/* Arguments of born_sample.  Pipeline per row: upcast -> penalties over the token
 * history -> grammar bitmask (-inf where the bit is 0) -> [greedy: first maximum] ->
 * top-k by (value desc, index asc) -> temperature -> min-p -> top-p -> inverse-CDF draw
 * in ascending token index with the caller's uniform. */
typedef struct born_sample_args {
    uint32_t struct_size; /* sizeof(born_sample_args) */
    uint32_t memory;      /* BORN_MEM_DEVICE or BORN_MEM_HOST */
    int32_t batch;
    int32_t vocab;
    int32_t logits_dtype; /* BORN_DTYPE_* */
    int32_t history_stride;    /* ids per row in `history` (<= BORN_MAX_HISTORY) */
    int64_t logits_row_stride; /* elements between rows (>= vocab) */
    const void* logits;        /* [batch, logits_row_stride] */
    const uint32_t* mask;      /* [batch, mask_row_stride] bitset, bit t&31 of word t>>5; NULL = none */
    int64_t mask_row_stride;   /* words between rows (>= ceil(vocab/32)) */
    const int32_t* history;     /* [batch, history_stride] prior token ids; ids outside [0,vocab) ignored; NULL = none */
    const int32_t* history_len; /* [batch] valid ids per row; NULL = history_stride */
    const born_row_params* row_params; /* [batch]; NULL = `params` for every row */
    born_row_params params;
    const float* uniforms; /* [batch] in [0,1); may be NULL when every row is greedy */
    int32_t* out_token;    /* [batch] */
    float* out_prob;       /* [batch] probability of the token within the kept set; NULL = skip */
    float* out_lse;        /* [batch] log-sum-exp of the scaled logits over the whole row; NULL = skip */
    int32_t* out_status;   /* [batch] BORN_ROW_* */
    int32_t* out_kept_ids;   /* [batch, kept_stride] kept set in rank order; NULL = skip */
    int32_t* out_kept_count; /* [batch]; NULL = skip */
    int32_t kept_stride;
    int32_t vocab_segments; /* 0/1 = off; G > 1: top-k is taken inside each of G equal contiguous
                               vocab segments (what a vocab-sharded lm_head produces) */
} born_sample_args;

/* Arguments of born_spec_verify (fp32 logits).  For position j = 0..draft_len-1: accept
 * draft token x_j iff u_accept * q_j(x_j) < p_j(x_j); at the first rejection draw from
 * max(0, p_j - q_j) and stop; if every position is accepted and target_rows ==
 * draft_len + 1, draw the bonus token from the last target row. */
typedef struct born_spec_args {
    uint32_t struct_size;
    uint32_t memory;
    int32_t batch;
    int32_t draft_len;   /* K <= BORN_MAX_DRAFT */
    int32_t vocab;
    int32_t target_rows; /* K or K+1 */
    const float* target_logits; /* [batch, target_rows, vocab] */
    const float* draft_logits;  /* [batch, K, vocab] */
    const int32_t* draft_tokens; /* [batch, K] */
    const float* u_accept;   /* [batch, K] */
    const float* u_resample; /* [batch, K+1]: entry j for a rejection at j, entry K for the bonus */
    float temperature;       /* 0 => 1 */
    int32_t reserved;
    int32_t* out_accept_len; /* [batch] */
    int32_t* out_tokens;     /* [batch, K+1] accepted tokens then the resampled/bonus token, -1 padded */
    int32_t* out_status;     /* [batch] */
} born_spec_args;

/* Arguments of the vocab-sharded path.  Every rank holds columns
 * [rank*vocab_local, (rank+1)*vocab_local) of every row.  born_shard_local writes one
 * packed record per row into `packed`; after an all-gather of those records
 * born_shard_merge draws the tokens; born_sample_sharded does all three. */
typedef struct born_shard_args {
    uint32_t struct_size;
    uint32_t memory; /* BORN_MEM_DEVICE only */
    int32_t batch;
    int32_t vocab_local;
    int32_t logits_dtype;
    int32_t rank;
    int32_t nranks;
    int32_t top_k;     /* per shard, 1..BORN_MAX_TOP_K/nranks */
    int64_t logits_row_stride;
    const void* logits; /* [batch, logits_row_stride] local shard */
    float temperature;
    float top_p;
    const float* uniforms; /* [batch]; identical on every rank */
    void* packed;      /* local pass out: [batch, born_shard_record_bytes(top_k)] */
    const void* gathered; /* merge in: [nranks, batch, record_bytes] */
    int32_t* out_token;
    float* out_prob;
    float* out_lse;
    int32_t* out_status;
} born_shard_args;

/* Replaces: nothing in the reference allocates device state; mirrors backend construction
 * cpu.New() (internal/backend/cpu/backend.go:16-20).  Allocates the workspace for up to
 * max_batch rows of max_vocab tokens on `device`.  Fails with BORN_ERR_NO_DEVICE when no
 * CUDA device is usable. */
int32_t born_sampler_create(int32_t device, int32_t max_batch, int32_t max_vocab, int32_t max_k, void** out_handle);
int32_t born_sampler_destroy(void* handle);

/* Replaces nn.Accuracy's per-row argmax (internal/nn/cross_entropy.go:241-284) and the
 * softmax / log-sum-exp row passes (internal/autodiff/ops/softmax.go:214-238,
 * internal/nn/cross_entropy.go:126-153) with the full sampling pipeline.  One kernel launch:
 * every logit is read once, whatever the parameters (per-row parameter arrays included).
 * Rows whose kept set is small (top-k, min-p, a nucleus of up to 1024 tokens) are finished
 * from the candidates collected while streaming; rows that nothing narrows are drawn from
 * exact per-512-token mass blocks; any other row (top-k above 256, a nucleus or a min-p
 * survivor set beyond 1024 tokens) takes an exact multi-pass search inside the same launch --
 * slower, never approximate.  Two more launches come first when whole-vocabulary rows are not
 * 16-byte aligned or are bf16 with history penalties (see "Ownership" above). */
int32_t born_sample(void* handle, const born_sample_args* args, void* stream);

/* No counterpart in the reference.  Allocates now whatever scratch a later born_sample call
 * with these arguments (same memory side, shapes, dtype, alignment and parameters) would
 * otherwise allocate on first use; runs nothing. */
int32_t born_sampler_reserve(void* handle, const born_sample_args* args);

/* No counterpart in the reference.  Reads and clears the handle's device error word
 * (synchronises the device).  Every on-device wait of the kernels is bounded; when one gives
 * up, the rows the CTA had a part in report row status 100 + BORN_ERR_DEVICE_TIMEOUT, and the
 * call is reported here -- BORN_MEM_HOST calls check by themselves and return
 * BORN_ERR_DEVICE_TIMEOUT, BORN_MEM_DEVICE calls are asynchronous and are checked with this. */
int32_t born_check_error(void* handle);

/* No counterpart in the reference (it has no speculative decoding); the row arithmetic is
 * the same max-shifted softmax as internal/autodiff/ops/softmax.go:214-238. */
int32_t born_spec_verify(void* handle, const born_spec_args* args, void* stream);

/* Vocab-sharded (tensor-parallel lm_head) sampling.  No counterpart in the reference
 * (distributed execution is a roadmap item there, ROADMAP.md:217-227). */
int32_t born_shard_record_bytes(int32_t top_k);
int32_t born_shard_unique_id(void* out_id128);  /* 128-byte NCCL unique id (rank 0) */
int32_t born_shard_init(void* handle, const void* nccl_unique_id, int32_t rank, int32_t nranks);
int32_t born_shard_local(void* handle, const born_shard_args* args, void* stream);
int32_t born_shard_merge(void* handle, const born_shard_args* args, void* stream);
int32_t born_sample_sharded(void* handle, const born_shard_args* args, void* stream);

/* No counterpart in the reference.  born_sample for callers that must not allocate device
 * memory -- code running where cudaMalloc is off limits (a pre-sized serving process whose
 * memory pool owns the whole GPU, a latency-critical decode loop, a host binding without a
 * place to keep a handle).  It needs no handle: the segment records, mass blocks and row
 * tickets the kernel uses as scratch live in a fixed array inside the library image, at most
 * BORN_STATIC_SCRATCH_BYTES per GPU that loads the library.  Limits, anything beyond them is
 * refused with BORN_ERR_UNSUPPORTED: device pointers only (BORN_MEM_DEVICE);
 * batch <= BORN_STATIC_MAX_BATCH; batch * ceil(vocab / 512) <= BORN_STATIC_MAX_BLOCKS; no
 * vocab_segments; and none of the calls that need the aligned fp32 copy (whole-vocabulary rows
 * -- no top-k and no min-p, or a per-row parameter array -- whose logits are not 16-byte
 * aligned or are bf16 with history penalties).  Runs on the current device.  The first call
 * on a device looks up the array's address; make that call before any stream capture.  All
 * calls on a device share the one array: calls that overlap on the GPU (different streams,
 * different threads) race and give wrong results -- serialise them.  Errors are reported
 * through born_last_error(NULL). */
#define BORN_STATIC_MAX_BATCH 256
#define BORN_STATIC_MAX_BLOCKS 131072
#define BORN_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
int32_t born_sample_static(const born_sample_args* args, void* stream);

/* No counterpart in the reference.  Rows that took the exact multi-pass search (see
 * born_sample) since the last call of this function; synchronises the device.  A serving
 * loop can watch it: a workload whose rows keep landing there is paying for a flat
 * distribution (or a top-k above 256), not for a fault. */
int64_t born_fallback_rows(void* handle);

/* Bytes of device workspace a handle holds (for capacity planning). */
int64_t born_workspace_bytes(void* handle);
/* Number of kernels the handle has launched since creation. */
int64_t born_launch_count(void* handle);
/* Device time of the last BORN_MEM_HOST call split as h2d / kernel / d2h, in ms. */
int32_t born_last_timing(void* handle, float* out3);

const char* born_last_error(void* handle);
const char* born_version(void);

/* Test hook: one small sampling launch in which one bulk copy is withheld and the wait limit
 * is a millisecond, so that the bounded wait gives up.  Returns BORN_ERR_DEVICE_TIMEOUT when
 * the kernel reported the expiry and came back (the expected outcome), BORN_OK when it did
 * not expire.  The handle stays usable.  Synchronises the stream. */
int32_t born_debug_expire_wait(void* handle, void* stream);

/* ---- the autoregressive loop around the sampler ---------------------------------------
 * The reference's only call site of this path is a per-batch loop on the host that takes the
 * arg-max of the model's output and compares it (examples/mnist/main.go:229-245); a language
 * model's generate loop does the same once per token, and feeds the token back.  The entry
 * points below keep what that loop carries from step to step on the device, so that step t+1
 * needs no host round trip for it.  None has a counterpart in the reference. */

/* Device-resident token history: per row the last `capacity` (<= BORN_MAX_HISTORY) tokens, a
 * count, and a finished flag.  Allocates for the handle's max_batch rows; calling it again
 * re-allocates.  Returns BORN_ERR_UNSUPPORTED for the handle of born_sample_static. */
int32_t born_history_create(void* handle, int32_t capacity);

/* Loads prompts: tokens [batch, stride] with lens [batch] valid ids per row (NULL: stride); only
 * the last `capacity` ids of a row are kept.  `memory` says where tokens/lens live.  Clears the
 * finished flags.  Ordered on `stream`. */
int32_t born_history_reset(void* handle, const int32_t* tokens, const int32_t* lens, int32_t batch, int32_t stride,
                           uint32_t memory, void* stream);

/* Up to 8 stop token ids (n = 0: none).  A row that samples one is reported normally in that
 * step and is finished from the next step on: token -1, status BORN_ROW_FINISHED, nothing
 * appended. */
int32_t born_history_set_stop_tokens(void* handle, const int32_t* ids, int32_t n);

/* Copies the state out (any pointer may be NULL): tokens [batch, capacity] in ring order (slot
 * i holds the (i mod capacity)-th token appended since the reset), total [batch] tokens
 * appended since the reset (prompt included), finished [batch].  Synchronises `stream`. */
int32_t born_history_read(void* handle, int32_t* tokens, int32_t* total, int32_t* finished, int32_t batch, uint32_t memory,
                          void* stream);

/* born_sample over the device-resident history: args->history and args->history_len must be
 * NULL, args->memory BORN_MEM_DEVICE, vocab_segments off.  The kernel that finishes a row
 * appends the sampled token to the row's history before it exits, so the next call sees it
 * with no host step in between. */
int32_t born_sample_next(void* handle, const born_sample_args* args, void* stream);

/* Grammar-mask producer interface (absent in the reference): two pinned host buffers and two
 * device buffers owned by the handle.  born_mask_begin hands out the pinned buffer to fill for
 * the next step ([batch, words_per_row] words, rows tight) while the previous step's kernel
 * may still be reading the other device buffer; born_mask_commit starts the copy to the
 * device on the handle's own copy stream and returns the device pointer to pass as
 * args->mask (mask_row_stride = words_per_row); born_mask_wait makes `stream` wait for that
 * copy (an event, no host synchronisation).  The first begin allocates; later ones re-allocate
 * only when batch * words_per_row grows. */
int32_t born_mask_begin(void* handle, int32_t batch, int32_t words_per_row, uint32_t** host_buffer);
int32_t born_mask_commit(void* handle, const uint32_t** device_mask);
int32_t born_mask_wait(void* handle, void* stream);

/* Test hooks: run the library's deterministic exp / fixed-point mass on device arrays. */
int32_t born_debug_exp(const float* x_dev, float* y_dev, int64_t n, void* stream);
int32_t born_debug_mass(const float* x_dev, uint64_t* q_dev, int64_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BORN_SAMPLER_H */
