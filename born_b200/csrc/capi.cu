// Host side of libborn_sampler.so: handle, argument checking, launch configuration and
// the host-memory convenience path.  Declarations and the reference interfaces each entry
// point stands in for are in include/born_sampler.h.
//
// Error split follows the reference's backend idiom (born: internal/backend/cpu/backend.go:35-37
// panics on programmer error, internal/tensor/raw.go:89-92 returns errors for expected
// failures): BORN_ERR_INVALID_ARGUMENT is the former, everything else the latter.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/born_sampler.h"
#include "scan_common.cuh"
#include "scan_launch.cuh"
#include "merge_kernel.cuh"
#include "prepass.cuh"
#include "spec_kernel.cuh"

using namespace born;

struct Id128 { char b[128]; };  // ncclUniqueId, passed by value to ncclCommInitRank

namespace {

struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, Id128, int) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};

struct Staging {  // device mirrors of host buffers for BORN_MEM_HOST calls
    void* p = nullptr;
    size_t bytes = 0;
};

struct Handle {
    int device = 0;
    int max_batch = 0, max_vocab = 0, max_k = 0;
    int num_sms = 0;
    int max_grid = 0;              // CTAs of the streaming kernel (two per SM)
    int max_rows = 0;              // virtual rows (caller rows x vocabulary segments) a call may stream
    int rec_cap = 0;               // entries per segment record
    int64_t rec_stride = 0;
    size_t records_bytes = 0;
    uint8_t* records = nullptr;    // segment records, indexed by row + cta
    MassBlock* blocks = nullptr;   // mass blocks of the whole-vocabulary routes
    int64_t blocks_cap = 0;
    uint32_t* tickets = nullptr;   // [max_rows] tickets, then [max_rows] deferred-fallback owners
    uint8_t* seg_packed = nullptr; // packed records of the one-GPU vocabulary-segment form
    size_t seg_packed_bytes = 0;
    int* dev_error = nullptr;
    unsigned long long timeout_ns = kMbarTimeoutNs;
    uint8_t* spec_scratch = nullptr;
    size_t spec_scratch_bytes = 0;
    int64_t spec_layout_key = -1;
    bool is_static = false;  // the handle of born_sample_static: may not allocate
    float* clean_copy = nullptr;  // aligned fp32 copy of the rows (mask and penalties applied)
    size_t clean_copy_bytes = 0;
    Staging stage[16];
    // device-resident history (born_history_*)
    int32_t* ring = nullptr;       // [max_batch, ring_cap], then total / len / finished [max_batch] each
    int ring_cap = 0;
    int n_stop = 0;
    int32_t stop_ids[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    bool use_ring = false;         // set by born_sample_next around its call of sample_device
    // grammar-mask upload (born_mask_*)
    uint32_t* mask_host[2] = {nullptr, nullptr};
    uint32_t* mask_dev[2] = {nullptr, nullptr};
    size_t mask_words = 0;         // words each of the four buffers holds
    size_t mask_pending_words = 0; // words of the buffer handed out by born_mask_begin
    int mask_next = 0;             // buffer the next born_mask_begin hands out
    int mask_filled = -1;          // buffer handed out and not yet committed
    cudaStream_t mask_stream = nullptr;
    cudaEvent_t mask_event = nullptr;
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
    float timing[3] = {0, 0, 0};
    int64_t launches = 0;
    int64_t workspace = 0;
    // vocab-sharded path
    NcclApi nccl;
    void* comm = nullptr;
    int rank = 0, nranks = 1;
    uint8_t* gathered = nullptr;
    size_t gathered_bytes = 0;
    uint8_t* packed = nullptr;
    size_t packed_bytes = 0;
    char err[512] = {0};
};

char g_err[512] = "";

int fail(Handle* h, int code, const char* fmt, ...) {
    char* dst = h ? h->err : g_err;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(dst, 512, fmt, ap);
    va_end(ap);
    return code;
}

#define CUDA_TRY(h, call)                                                                      \
    do {                                                                                       \
        cudaError_t e_ = (call);                                                               \
        if (e_ != cudaSuccess)                                                                 \
            return fail(h, BORN_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_));     \
    } while (0)

int dev_alloc(Handle* h, void** p, size_t bytes) {
    if (h->is_static) return fail(h, BORN_ERR_UNSUPPORTED, "this call needs %zu bytes of scratch that the allocation-free entry point may not allocate", bytes);
    cudaError_t e = cudaMalloc(p, bytes);
    if (e != cudaSuccess) return fail(h, BORN_ERR_CUDA, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    h->workspace += (int64_t)bytes;
    return BORN_OK;
}

// Grow-only scratch: allocated at the size of the largest request seen (born_sampler_reserve
// makes that request ahead of time), never per call afterwards.
int grow(Handle* h, void** p, size_t* have, size_t need, cudaStream_t st) {
    if (*have >= need) return BORN_OK;
    if (h->is_static) return fail(h, BORN_ERR_UNSUPPORTED, "this call needs %zu bytes of scratch that the allocation-free entry point may not allocate", need);
    if (*p) {
        cudaError_t e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) return fail(h, BORN_ERR_CUDA, "cudaStreamSynchronize failed: %s", cudaGetErrorString(e));
        cudaFree(*p);
        h->workspace -= (int64_t)*have;
        *p = nullptr;
        *have = 0;
    }
    int rc = dev_alloc(h, p, need);
    if (rc == BORN_OK) *have = need;
    return rc;
}

int stage_reserve(Handle* h, int slot, size_t bytes) {
    Staging& s = h->stage[slot];
    return grow(h, &s.p, &s.bytes, bytes, nullptr);
}

int use_device(Handle* h) {
    int cur = -1;
    if (cudaGetDevice(&cur) == cudaSuccess && cur == h->device) return BORN_OK;
    CUDA_TRY(h, cudaSetDevice(h->device));
    return BORN_OK;
}

bool params_ok(const born_row_params& p) {
    if (!(p.temperature >= 0.0f) || !isfinite(p.temperature)) return false;
    if (p.temperature != 0.0f && p.temperature < 1e-4f) return false;
    if (!(p.top_p >= 0.0f) || !isfinite(p.top_p)) return false;
    if (!(p.min_p >= 0.0f) || p.min_p > 1.0f) return false;
    if (p.top_k < 0 || p.top_k > BORN_MAX_TOP_K) return false;
    if (!(p.repetition_penalty >= 0.0f) || !isfinite(p.repetition_penalty)) return false;
    if (!isfinite(p.frequency_penalty) || !isfinite(p.presence_penalty)) return false;
    return true;
}

bool host_penalties_on(const born_row_params& p) {
    return (p.repetition_penalty != 1.0f && p.repetition_penalty != 0.0f) || p.frequency_penalty != 0.0f ||
           p.presence_penalty != 0.0f;
}
// no top-k and no min-p: the row total comes from the mass blocks (temperature-only, top-p alone)
bool host_need_mass(const born_row_params& p) {
    const bool greedy = (p.flags & BORN_FLAG_GREEDY) || p.temperature == 0.0f;
    return !greedy && p.top_k <= 0 && !(p.min_p > 0.0f);
}

// The dynamic shared-memory limit of every instantiation is raised once (at create / first static call).
cudaError_t scan_attrs_all() {
    cudaError_t e;
    if ((e = scan_attrs_f32_pair()) != cudaSuccess) return e;
    if ((e = scan_attrs_f32_pair_row()) != cudaSuccess) return e;
    if ((e = scan_attrs_f32_hist()) != cudaSuccess) return e;
    if ((e = scan_attrs_f32_hist_row()) != cudaSuccess) return e;
    if ((e = scan_attrs_f32_hist_short_row()) != cudaSuccess) return e;
    if ((e = scan_attrs_bf16_pair()) != cudaSuccess) return e;
    if ((e = scan_attrs_bf16_pair_row()) != cudaSuccess) return e;
    if ((e = scan_attrs_bf16()) != cudaSuccess) return e;
    return scan_attrs_bf16_row();
}

// The route class of a launch (RouteOf in scan_common.cuh): uniform parameters tell it on the host.
static int route_of(const born_row_params* row_params, const born_row_params& p) {
    if (row_params) return 0;
    if (host_need_mass(p)) return 0;
    const bool greedy = (p.flags & BORN_FLAG_GREEDY) || p.temperature == 0.0f;
    return (!greedy && p.top_k > 0) ? 2 : 1;
}

int launch_scan(Handle* h, const ScanArgs& A, int dtype, int grid, cudaStream_t st) {
    const int route = route_of(A.row_params, A.params);
    const bool has_mask = A.mask != nullptr;
    const bool lse = A.out_lse != nullptr || A.want_lse;

    // Launches without a token history take the instantiations that carry no history code (fp32:
    // their loop pairs tiles); launches with one take the others.
    // A sampling launch whose grid is one CTA per row (the tile ranges of range_begin are then the
    // rows themselves) takes the instantiations without the segment-record path.
    const bool one_row = A.mode == kScanFull && A.G == 1 && grid == A.B;
    // ... and, fp32 with histories of at most kHistShort ids per row, the one whose list takes half the room
    const bool short_hist = one_row && dtype == BORN_DTYPE_F32 && A.history != nullptr && A.history_stride <= kHistShort;
    const size_t smem = (size_t)scan_smem_layout(dtype == BORN_DTYPE_F32 ? 4 : 2, has_mask, A.history != nullptr,
                                                 short_hist ? kHistShort : (int)BORN_MAX_HISTORY).total;
    cudaError_t e;
    if (dtype != BORN_DTYPE_F32 && A.history == nullptr)
        e = one_row ? scan_launch_bf16_pair_row(A, has_mask, lse, route, grid, smem, st)
                    : scan_launch_bf16_pair(A, has_mask, lse, route, grid, smem, st);
    else if (dtype != BORN_DTYPE_F32)
        e = one_row ? scan_launch_bf16_row(A, has_mask, lse, route, grid, smem, st) : scan_launch_bf16(A, has_mask, lse, route, grid, smem, st);
    else if (A.history == nullptr)
        e = one_row ? scan_launch_f32_pair_row(A, has_mask, lse, route, grid, smem, st)
                    : scan_launch_f32_pair(A, has_mask, lse, route, grid, smem, st);
    else
        e = short_hist ? scan_launch_f32_hist_short_row(A, has_mask, lse, route, grid, smem, st)
            : one_row  ? scan_launch_f32_hist_row(A, has_mask, lse, route, grid, smem, st)
                       : scan_launch_f32_hist(A, has_mask, lse, route, grid, smem, st);
    if (e != cudaSuccess) return fail(h, BORN_ERR_CUDA, "scan kernel launch failed: %s", cudaGetErrorString(e));
    h->launches++;
    return BORN_OK;
}

int launch_merge(Handle* h, const MergeArgs& M, cudaStream_t st) {
    merge_kernel<<<M.B, kThreads, 2 * kSelCap * 8, st>>>(M);
    CUDA_TRY(h, cudaGetLastError());
    h->launches++;
    return BORN_OK;
}

// Geometry and scratch of one streaming launch over B x G virtual rows of V tokens.
int fill_scan(Handle* h, ScanArgs& A, int B, int G, int V, int dtype, const void* logits, int64_t row_stride,
              const uint32_t* mask, int64_t mask_stride, int* grid) {
    const int esz = dtype == BORN_DTYPE_F32 ? 4 : 2;
    if ((uintptr_t)logits % esz) return fail(h, BORN_ERR_INVALID_ARGUMENT, "logits pointer is not aligned to its element size");
    if (mask && (uintptr_t)mask % 4) return fail(h, BORN_ERR_INVALID_ARGUMENT, "mask pointer is not 4-byte aligned");
    bool fast = ((uintptr_t)logits % 16 == 0) && ((row_stride * esz) % 16 == 0) && (G == 1 || ((int64_t)V * esz) % 16 == 0);
    if (mask) fast = fast && ((uintptr_t)mask % 16 == 0) && ((mask_stride * 4) % 16 == 0) && (G == 1 || V % 128 == 0);
    const int tile = kTileBytes / esz;
    const int lead_max = fast ? 0 : 16 / esz - 1;
    A.B = B; A.G = G; A.V = V;
    A.tpr = (int)(((int64_t)V + lead_max + tile - 1) / tile);
    A.fast = fast ? 1 : 0;
    A.logits = logits; A.row_stride = row_stride;
    A.mask = mask; A.mask_stride = mask_stride;
    const int64_t rows = (int64_t)B * G;
    if (rows > h->max_rows) return fail(h, BORN_ERR_UNSUPPORTED, "%lld rows (batch x segments) exceed the workspace of %d", (long long)rows, h->max_rows);
    A.nblk = (V + kMassBlock - 1) / kMassBlock;
    if (rows * A.nblk > h->blocks_cap) return fail(h, BORN_ERR_UNSUPPORTED, "batch x vocab exceeds the workspace");
    const int64_t tiles = rows * A.tpr;
    *grid = (int)(tiles < h->max_grid ? tiles : h->max_grid);
    // When a whole number S of equal slices per row nearly fills the GPU, every CTA gets exactly
    // one slice: no CTA meets a row boundary in mid-stream, and with S = 1 a row is finished from
    // the shared memory of the CTA that streamed it.
    for (int S = 1; S <= 64 && rows * S <= h->max_grid; ++S)
        if (A.tpr % S == 0 && rows * S * 20 >= (int64_t)h->max_grid * 17) { *grid = (int)(rows * S); break; }
    // entries per segment record: as many as the record area gives every (row + cta) slot
    int64_t cap = ((int64_t)(h->records_bytes / (size_t)(rows + *grid)) - kRecordHdrBytes) / 8;
    cap = (cap < h->rec_cap ? cap : h->rec_cap) & ~(int64_t)1;
    if (cap < 64) return fail(h, BORN_ERR_UNSUPPORTED, "%lld rows (batch x segments) exceed the record workspace", (long long)rows);
    A.records = h->records; A.rec_cap = (int)cap; A.rec_stride = kRecordHdrBytes + cap * 8;
    A.blocks = h->blocks;
    A.tickets = h->tickets; A.deferred = h->tickets + h->max_rows;
    A.dev_error = h->dev_error;
    A.timeout_ns = h->timeout_ns;
    A.debug_skip_tile = -1;
    return BORN_OK;
}

int check_device_error(Handle* h) {
    int e = 0;
    CUDA_TRY(h, cudaMemcpy(&e, h->dev_error, sizeof(int), cudaMemcpyDeviceToHost));
    if (e) {
        // tickets of rows that were left unfinished must not leak into the next launch
        cudaMemset(h->tickets, 0, sizeof(uint32_t) * 2 * (size_t)h->max_rows);
        cudaMemset(h->dev_error, 0, sizeof(int));
        return fail(h, BORN_ERR_DEVICE_TIMEOUT, "a bounded on-device wait gave up (code %d); outputs of that call are invalid", e);
    }
    return BORN_OK;
}

__global__ void debug_exp_kernel(const float* x, float* y, int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = exp_det(x[i]);
}
__global__ void debug_mass_kernel(const float* x, unsigned long long* q, int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) q[i] = mass_of(x[i]);
}

// scratch sizes of a handle for max_batch rows of max_vocab tokens
struct ScratchPlan {
    int max_rows, rec_cap;
    int64_t rec_stride, blocks_cap;
    size_t records, blocks, tickets, seg_packed, hist, total;
};
ScratchPlan scratch_plan(int max_batch, int max_vocab, int max_grid, int rec_cap) {
    ScratchPlan p;
    // virtual rows (caller rows x vocabulary segments); the record area is sized for full-size
    // records of 2 * max_batch rows and is cut finer when a call streams more rows than that
    p.max_rows = max_batch * BORN_MAX_SHARDS > 1024 ? max_batch * BORN_MAX_SHARDS : 1024;
    p.rec_cap = rec_cap;
    p.rec_stride = kRecordHdrBytes + (int64_t)rec_cap * 8;
    p.records = (size_t)((max_batch * 2 > 1024 ? max_batch * 2 : 1024) + max_grid) * (size_t)p.rec_stride;
    // a call of B x G rows of V tokens needs B*G*ceil(V/512) blocks; segments only shorten V
    p.blocks_cap = (int64_t)max_batch * (((int64_t)max_vocab + kMassBlock - 1) / kMassBlock) + p.max_rows;
    p.blocks = (size_t)p.blocks_cap * sizeof(MassBlock);
    p.tickets = sizeof(uint32_t) * 2 * (size_t)p.max_rows;
    p.seg_packed = (size_t)max_batch * (size_t)(kRecordHdrBytes * BORN_MAX_SHARDS + 8 * BORN_MAX_CANDIDATES);
    p.total = p.records + p.blocks + p.tickets + p.seg_packed + 256;
    return p;
}

}  // namespace

extern "C" {

const char* born_version(void) { return "born-sampler-b200 0.2.0 (sm_100a)"; }

const char* born_last_error(void* handle) { return handle ? ((Handle*)handle)->err : g_err; }

int32_t born_sampler_create(int32_t device, int32_t max_batch, int32_t max_vocab, int32_t max_k, void** out) {
    if (!out) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "out_handle is NULL");
    *out = nullptr;
    if (max_batch <= 0 || max_vocab <= 0 || max_vocab > BORN_MAX_VOCAB || max_k < 0 || max_k > BORN_MAX_TOP_K)
        return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "create: max_batch=%d max_vocab=%d max_k=%d out of range",
                    max_batch, max_vocab, max_k);
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev <= 0)
        return fail(nullptr, BORN_ERR_NO_DEVICE, "no CUDA device: %s (this library has no CPU path)",
                    e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    if (device < 0 || device >= ndev)
        return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "device %d out of range (have %d)", device, ndev);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess)
        return fail(nullptr, BORN_ERR_CUDA, "cudaGetDeviceProperties failed");
    if (prop.major != 10)
        return fail(nullptr, BORN_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                    prop.major, prop.minor);
    Handle* h = new Handle();
    h->device = device;
    h->max_batch = max_batch;
    h->max_vocab = max_vocab;
    h->max_k = max_k > 0 ? max_k : BORN_MAX_TOP_K;
    h->num_sms = prop.multiProcessorCount;
    h->max_grid = 2 * h->num_sms;
    if (cudaSetDevice(device) != cudaSuccess) { delete h; return fail(nullptr, BORN_ERR_CUDA, "cudaSetDevice failed"); }
    const ScratchPlan sp = scratch_plan(max_batch, max_vocab, h->max_grid, 2048);
    h->max_rows = sp.max_rows;
    h->rec_cap = sp.rec_cap;
    h->rec_stride = sp.rec_stride;
    h->records_bytes = sp.records;
    h->blocks_cap = sp.blocks_cap;
    h->seg_packed_bytes = sp.seg_packed;
    int rc = dev_alloc(h, (void**)&h->records, sp.records);
    if (rc == BORN_OK) rc = dev_alloc(h, (void**)&h->blocks, sp.blocks);
    if (rc == BORN_OK) rc = dev_alloc(h, (void**)&h->tickets, sp.tickets);
    if (rc == BORN_OK) rc = dev_alloc(h, (void**)&h->seg_packed, sp.seg_packed);
    if (rc == BORN_OK) rc = dev_alloc(h, (void**)&h->dev_error, 32 * sizeof(int));
    if (rc == BORN_OK && cudaMemset(h->tickets, 0, sp.tickets) != cudaSuccess) rc = BORN_ERR_CUDA;
    if (rc == BORN_OK && cudaMemset(h->dev_error, 0, 32 * sizeof(int)) != cudaSuccess) rc = BORN_ERR_CUDA;
    if (rc == BORN_OK && scan_attrs_all() != cudaSuccess) rc = BORN_ERR_CUDA;
    if (rc == BORN_OK && spec_attrs_all() != cudaSuccess) rc = BORN_ERR_CUDA;
    for (int i = 0; i < 4 && rc == BORN_OK; ++i)
        if (cudaEventCreate(&h->ev[i]) != cudaSuccess) rc = BORN_ERR_CUDA;
    if (rc != BORN_OK) {
        snprintf(g_err, sizeof g_err, "create failed: %.480s", h->err[0] ? h->err : cudaGetErrorString(cudaGetLastError()));
        born_sampler_destroy(h);
        return rc;
    }
    *out = h;
    return BORN_OK;
}

int32_t born_sampler_destroy(void* handle) {
    Handle* h = (Handle*)handle;
    if (!h) return BORN_OK;
    cudaSetDevice(h->device);
    if (h->comm && h->nccl.CommDestroy) h->nccl.CommDestroy(h->comm);
    cudaFree(h->ring);
    for (int i = 0; i < 2; ++i) {
        if (h->mask_host[i]) cudaFreeHost(h->mask_host[i]);
        cudaFree(h->mask_dev[i]);
    }
    if (h->mask_stream) cudaStreamDestroy(h->mask_stream);
    if (h->mask_event) cudaEventDestroy(h->mask_event);
    cudaFree(h->records);
    cudaFree(h->blocks);
    cudaFree(h->tickets);
    cudaFree(h->seg_packed);
    cudaFree(h->dev_error);
    cudaFree(h->spec_scratch);
    cudaFree(h->clean_copy);
    cudaFree(h->gathered);
    cudaFree(h->packed);
    for (auto& s : h->stage) cudaFree(s.p);
    for (auto& e : h->ev) if (e) cudaEventDestroy(e);
    delete h;
    return BORN_OK;
}

int64_t born_workspace_bytes(void* handle) { return handle ? ((Handle*)handle)->workspace : 0; }
int64_t born_launch_count(void* handle) { return handle ? ((Handle*)handle)->launches : 0; }
int32_t born_last_timing(void* handle, float* out3) {
    if (!handle || !out3) return BORN_ERR_INVALID_ARGUMENT;
    memcpy(out3, ((Handle*)handle)->timing, sizeof(float) * 3);
    return BORN_OK;
}

int64_t born_fallback_rows(void* handle) {
    Handle* h = (Handle*)handle;
    if (!h || h->is_static) return -1;
    if (use_device(h)) return -1;
    int n[24];
    if (cudaMemcpy(n, h->dev_error + 1, sizeof n, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    cudaMemset(h->dev_error + 1, 0, sizeof n);
    // by reason: 1 greedy tie lost, 2 kept-id list of a whole row, 3 more than 1024 candidates, 4 top-k above 256,
    // 5 / 6 top-k / min-p set not provably complete, 7 nucleus below the candidates, 8 shard record not exact
    snprintf(h->err, sizeof h->err, "exact-search rows by reason 1..8: %d %d %d %d %d %d %d %d", n[8], n[9], n[10], n[11], n[12],
             n[13], n[14], n[15]);
    return n[0];
}

int32_t born_check_error(void* handle) {
    Handle* h = (Handle*)handle;
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    if (h->is_static) return BORN_ERR_INVALID_ARGUMENT;
    int rc = use_device(h);
    if (rc) return rc;
    return check_device_error(h);
}

// Does this call have to go through the clean fp32 copy first?  Only rows whose total comes
// from the mass blocks are concerned (no top-k, no min-p); with per-row parameter arrays on
// the device the host cannot tell, so it assumes that some row is.
static bool wants_clean_copy(const born_sample_args* a, bool fast) {
    if (a->vocab_segments > 1) return false;  // segments need top-k
    const bool may_mass = a->row_params ? true : host_need_mass(a->params);
    if (!may_mass) return false;
    if (!fast) return true;
    const bool pen = a->history && (a->row_params ? true : host_penalties_on(a->params));
    return pen && a->logits_dtype == BORN_DTYPE_BF16;
}

static int sample_device(Handle* h, const born_sample_args* a_in, cudaStream_t st, bool reserve_only) {
    const born_sample_args* a = a_in;
    born_sample_args a2;
    ScanArgs A;
    memset(&A, 0, sizeof A);
    int grid = 0;
    const int G = a->vocab_segments > 1 ? a->vocab_segments : 1;
    int rc = fill_scan(h, A, a->batch, G, a->vocab / G, a->logits_dtype, a->logits, a->logits_row_stride, a->mask,
                       a->mask_row_stride, &grid);
    if (rc) return rc;
    if (wants_clean_copy(a, A.fast != 0)) {
        const int64_t v_pad = ((int64_t)a->vocab + 3) / 4 * 4;
        const size_t need = (size_t)a->batch * (size_t)v_pad * sizeof(float);
        if ((rc = grow(h, (void**)&h->clean_copy, &h->clean_copy_bytes, need, st))) return rc;
        if (!reserve_only) {
            CopyArgs C;
            memset(&C, 0, sizeof C);
            C.logits = a->logits; C.out = h->clean_copy; C.mask = a->mask;
            C.history = a->history; C.history_len = a->history_len; C.history_stride = a->history_stride;
            C.row_params = a->row_params; C.params = a->params;
            C.row_stride = a->logits_row_stride; C.out_stride = v_pad; C.mask_stride = a->mask_row_stride;
            C.B = a->batch; C.V = a->vocab;
            int nl = 0;
            const int e = launch_clean_copy(C, a->logits_dtype, h->num_sms, st, &nl);
            h->launches += nl;
            if (e != 0) return fail(h, BORN_ERR_CUDA, "clean-copy launch failed: %s", cudaGetErrorString((cudaError_t)e));
        }
        a2 = *a;
        a2.logits = h->clean_copy; a2.logits_dtype = BORN_DTYPE_F32; a2.logits_row_stride = v_pad;
        a2.mask = nullptr; a2.mask_row_stride = 0;
        a2.history = nullptr; a2.history_len = nullptr; a2.history_stride = 0;
        a = &a2;
        rc = fill_scan(h, A, a->batch, 1, a->vocab, a->logits_dtype, a->logits, a->logits_row_stride, nullptr, 0, &grid);
        if (rc) return rc;
    }
    if (reserve_only) return BORN_OK;
    A.history = a->history;
    A.history_len = a->history_len;
    A.history_stride = a->history_stride;
    if (h->use_ring) {
        int32_t* meta = h->ring + (size_t)h->max_batch * h->ring_cap;
        A.ring = h->ring;
        A.ring_total = meta;
        A.ring_len = meta + h->max_batch;
        A.ring_finished = meta + 2 * (size_t)h->max_batch;
        A.ring_cap = h->ring_cap;
        A.n_stop = h->n_stop;
        memcpy(A.stop_ids, h->stop_ids, sizeof A.stop_ids);
    }
    A.row_params = a->row_params;
    A.params = a->params;
    A.uniforms = a->uniforms;
    A.out_token = a->out_token;
    A.out_prob = a->out_prob;
    A.out_lse = a->out_lse;
    A.out_status = a->out_status;
    A.out_kept_ids = a->out_kept_ids;
    A.out_kept_count = a->out_kept_count;
    A.kept_stride = a->kept_stride;
    A.mode = kScanFull;
    if (G > 1) {
        // vocabulary segments on one GPU: the k best of every (row, segment), then the merge --
        // the same two steps as the vocab-sharded path, without the all-gather in between
        const int64_t rec = kRecordHdrBytes + 8 * (int64_t)a->params.top_k;
        A.mode = kScanLocal;
        A.want_lse = a->out_lse != nullptr;
        A.out_lse = nullptr;
        A.packed = h->seg_packed;
        A.packed_row_stride = rec;
        A.packed_seg_stride = rec * a->batch;
        if ((size_t)(rec * a->batch * G) > h->seg_packed_bytes) return fail(h, BORN_ERR_UNSUPPORTED, "batch x segments x top_k exceeds the workspace");
        if ((rc = launch_scan(h, A, a->logits_dtype, grid, st))) return rc;
        MergeArgs M;
        memset(&M, 0, sizeof M);
        M.gathered = h->seg_packed; M.row_stride = rec; M.seg_stride = rec * a->batch;
        M.B = a->batch; M.G = G;
        M.temperature = a->params.temperature; M.top_p = a->params.top_p;
        M.uniforms = a->uniforms;
        M.out_token = a->out_token; M.out_prob = a->out_prob; M.out_lse = a->out_lse; M.out_status = a->out_status;
        M.out_kept_ids = a->out_kept_ids; M.out_kept_count = a->out_kept_count; M.kept_stride = a->kept_stride;
        return launch_merge(h, M, st);
    }
    return launch_scan(h, A, a->logits_dtype, grid, st);
}

static int sample_check(Handle* h, const born_sample_args* a) {
    if (!a) return fail(h, BORN_ERR_INVALID_ARGUMENT, "args is NULL");
    if (a->struct_size != sizeof(born_sample_args))
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "struct_size %u != %zu", a->struct_size, sizeof(born_sample_args));
    if (a->batch <= 0 || a->vocab <= 0) return fail(h, BORN_ERR_INVALID_ARGUMENT, "batch and vocab must be positive");
    if (a->batch > h->max_batch || a->vocab > h->max_vocab)
        return fail(h, h->is_static ? BORN_ERR_UNSUPPORTED : BORN_ERR_INVALID_ARGUMENT,
                    "batch %d / vocab %d exceed the limit of %d / %d", a->batch, a->vocab, h->max_batch, h->max_vocab);
    if (a->logits_dtype != BORN_DTYPE_F32 && a->logits_dtype != BORN_DTYPE_BF16)
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "unknown logits_dtype %d", a->logits_dtype);
    if (!a->logits || !a->out_token || !a->out_status)
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "logits, out_token and out_status are required");
    if (a->logits_row_stride < a->vocab) return fail(h, BORN_ERR_INVALID_ARGUMENT, "logits_row_stride < vocab");
    if (a->mask && a->mask_row_stride < (a->vocab + 31) / 32)
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "mask_row_stride < ceil(vocab/32)");
    if (a->history && (a->history_stride <= 0 || a->history_stride > BORN_MAX_HISTORY))
        return fail(h, a->history_stride > BORN_MAX_HISTORY ? BORN_ERR_UNSUPPORTED : BORN_ERR_INVALID_ARGUMENT,
                    "history_stride %d outside 1..%d", a->history_stride, BORN_MAX_HISTORY);
    if (a->memory != BORN_MEM_DEVICE && a->memory != BORN_MEM_HOST)
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "memory must be BORN_MEM_DEVICE or BORN_MEM_HOST");
    if (a->out_kept_ids && (a->kept_stride <= 0 || a->kept_stride > BORN_MAX_CANDIDATES))
        return fail(h, a->kept_stride > BORN_MAX_CANDIDATES ? BORN_ERR_UNSUPPORTED : BORN_ERR_INVALID_ARGUMENT,
                    "kept_stride must be in 1..%d", BORN_MAX_CANDIDATES);
    bool need_u = true;
    if (!a->row_params || a->memory == BORN_MEM_HOST) {
        const born_row_params* rp = a->row_params ? a->row_params : &a->params;
        const int n = a->row_params ? a->batch : 1;
        need_u = false;
        for (int i = 0; i < n; ++i) {
            if (!params_ok(rp[i])) return fail(h, BORN_ERR_INVALID_ARGUMENT, "sampling parameters of row %d out of range", i);
            if (!((rp[i].flags & BORN_FLAG_GREEDY) || rp[i].temperature == 0.0f)) need_u = true;
        }
    }
    if (need_u && !a->uniforms) return fail(h, BORN_ERR_INVALID_ARGUMENT, "uniforms required unless every row is greedy");
    if (a->vocab_segments > 1) {
        const int G = a->vocab_segments;
        if (G > BORN_MAX_SHARDS || a->vocab % G) return fail(h, BORN_ERR_INVALID_ARGUMENT, "vocab_segments must divide vocab and be <= %d", BORN_MAX_SHARDS);
        if (a->row_params) return fail(h, BORN_ERR_UNSUPPORTED, "vocab_segments needs uniform parameters");
        if (a->params.top_k <= 0 || a->params.top_k * G > BORN_MAX_CANDIDATES)
            return fail(h, BORN_ERR_UNSUPPORTED, "vocab_segments needs 1 <= top_k*segments <= %d", BORN_MAX_CANDIDATES);
        if (a->params.top_k > kThreads) return fail(h, BORN_ERR_UNSUPPORTED, "vocab_segments needs top_k <= %d per segment", kThreads);
        if ((a->params.flags & BORN_FLAG_GREEDY) || a->params.temperature == 0.0f || a->params.min_p > 0.0f)
            return fail(h, BORN_ERR_UNSUPPORTED, "vocab_segments takes temperature > 0, top-k and top-p only");
        if ((int64_t)G * a->batch > h->max_rows) return fail(h, BORN_ERR_UNSUPPORTED, "batch*segments exceeds the workspace");
        if (h->is_static) return fail(h, BORN_ERR_UNSUPPORTED, "vocab_segments needs scratch that the allocation-free entry point does not have");
    }
    return BORN_OK;
}

int32_t born_sampler_reserve(void* handle, const born_sample_args* a) {
    Handle* h = (Handle*)handle;
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    int rc = sample_check(h, a);
    if (rc) return rc;
    if ((rc = use_device(h))) return rc;
    if (a->memory == BORN_MEM_HOST) {
        const int B = a->batch, V = a->vocab;
        const size_t esz = a->logits_dtype == BORN_DTYPE_F32 ? 4 : 2;
        const size_t v_pad = ((size_t)V * esz + 15) / 16 * 16 / esz, w_pad = ((size_t)(V + 31) / 32 + 3) / 4 * 4;
        if ((rc = stage_reserve(h, 0, (size_t)B * v_pad * esz))) return rc;
        if (a->mask && (rc = stage_reserve(h, 1, (size_t)B * w_pad * 4))) return rc;
        if (a->history && (rc = stage_reserve(h, 2, (size_t)B * a->history_stride * 4))) return rc;
        for (int s = 3; s <= 11; ++s) {
            size_t need = (size_t)B * (s == 4 ? sizeof(born_row_params) : s == 10 ? (size_t)(a->kept_stride > 0 ? a->kept_stride : 1) * 4 : 4);
            if ((rc = stage_reserve(h, s, need))) return rc;
        }
        // the device form of the call: aligned staging rows
        born_sample_args d = *a;
        d.memory = BORN_MEM_DEVICE;
        d.logits = h->stage[0].p; d.logits_row_stride = (int64_t)v_pad;
        if (a->mask) { d.mask = (const uint32_t*)h->stage[1].p; d.mask_row_stride = (int64_t)w_pad; }
        return sample_device(h, &d, nullptr, true);
    }
    return sample_device(h, a, nullptr, true);
}

int32_t born_sample(void* handle, const born_sample_args* a, void* stream) {
    Handle* h = (Handle*)handle;
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    int rc = sample_check(h, a);
    if (rc) return rc;
    if ((rc = use_device(h))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (a->memory == BORN_MEM_DEVICE) return sample_device(h, a, st, false);

    // ---- host-memory call: copy in, run, copy out, wait ----
    const int B = a->batch, V = a->vocab;
    const size_t esz = a->logits_dtype == BORN_DTYPE_F32 ? 4 : 2;
    const size_t words = (size_t)(V + 31) / 32;
    born_sample_args d = *a;
    d.memory = BORN_MEM_DEVICE;
    // tight device copies: row strides become vocab (padded to 16 bytes)
    const size_t v_pad = ((size_t)V * esz + 15) / 16 * 16 / esz;
    const size_t w_pad = (words + 3) / 4 * 4;
    if ((rc = stage_reserve(h, 0, (size_t)B * v_pad * esz))) return rc;
    if (a->mask && (rc = stage_reserve(h, 1, (size_t)B * w_pad * 4))) return rc;
    if (a->history && (rc = stage_reserve(h, 2, (size_t)B * a->history_stride * 4))) return rc;
    if (a->history_len && (rc = stage_reserve(h, 3, (size_t)B * 4))) return rc;
    if (a->row_params && (rc = stage_reserve(h, 4, (size_t)B * sizeof(born_row_params)))) return rc;
    if (a->uniforms && (rc = stage_reserve(h, 5, (size_t)B * 4))) return rc;
    if ((rc = stage_reserve(h, 6, (size_t)B * 4))) return rc;
    if ((rc = stage_reserve(h, 7, (size_t)B * 4))) return rc;
    if ((rc = stage_reserve(h, 8, (size_t)B * 4))) return rc;
    if ((rc = stage_reserve(h, 9, (size_t)B * 4))) return rc;
    if (a->out_kept_ids && (rc = stage_reserve(h, 10, (size_t)B * a->kept_stride * 4))) return rc;
    if ((rc = stage_reserve(h, 11, (size_t)B * 4))) return rc;

    CUDA_TRY(h, cudaEventRecord(h->ev[0], st));
    CUDA_TRY(h, cudaMemcpy2DAsync(h->stage[0].p, v_pad * esz, a->logits, (size_t)a->logits_row_stride * esz,
                                  (size_t)V * esz, B, cudaMemcpyHostToDevice, st));
    d.logits = h->stage[0].p;
    d.logits_row_stride = (int64_t)v_pad;
    if (a->mask) {
        CUDA_TRY(h, cudaMemcpy2DAsync(h->stage[1].p, w_pad * 4, a->mask, (size_t)a->mask_row_stride * 4, words * 4, B,
                                      cudaMemcpyHostToDevice, st));
        d.mask = (const uint32_t*)h->stage[1].p;
        d.mask_row_stride = (int64_t)w_pad;
    }
    if (a->history) {
        CUDA_TRY(h, cudaMemcpyAsync(h->stage[2].p, a->history, (size_t)B * a->history_stride * 4, cudaMemcpyHostToDevice, st));
        d.history = (const int32_t*)h->stage[2].p;
    }
    if (a->history_len) {
        CUDA_TRY(h, cudaMemcpyAsync(h->stage[3].p, a->history_len, (size_t)B * 4, cudaMemcpyHostToDevice, st));
        d.history_len = (const int32_t*)h->stage[3].p;
    }
    if (a->row_params) {
        CUDA_TRY(h, cudaMemcpyAsync(h->stage[4].p, a->row_params, (size_t)B * sizeof(born_row_params), cudaMemcpyHostToDevice, st));
        d.row_params = (const born_row_params*)h->stage[4].p;
    }
    if (a->uniforms) {
        CUDA_TRY(h, cudaMemcpyAsync(h->stage[5].p, a->uniforms, (size_t)B * 4, cudaMemcpyHostToDevice, st));
        d.uniforms = (const float*)h->stage[5].p;
    }
    d.out_token = (int32_t*)h->stage[6].p;
    d.out_prob = a->out_prob ? (float*)h->stage[7].p : nullptr;
    d.out_lse = a->out_lse ? (float*)h->stage[8].p : nullptr;
    d.out_status = (int32_t*)h->stage[9].p;
    d.out_kept_ids = a->out_kept_ids ? (int32_t*)h->stage[10].p : nullptr;
    d.out_kept_count = a->out_kept_count ? (int32_t*)h->stage[11].p : nullptr;
    if (d.out_kept_ids) CUDA_TRY(h, cudaMemsetAsync(d.out_kept_ids, 0xFF, (size_t)B * a->kept_stride * 4, st));
    CUDA_TRY(h, cudaEventRecord(h->ev[1], st));
    if ((rc = sample_device(h, &d, st, false))) return rc;
    CUDA_TRY(h, cudaEventRecord(h->ev[2], st));
    CUDA_TRY(h, cudaMemcpyAsync(a->out_token, d.out_token, (size_t)B * 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(h, cudaMemcpyAsync(a->out_status, d.out_status, (size_t)B * 4, cudaMemcpyDeviceToHost, st));
    if (a->out_prob) CUDA_TRY(h, cudaMemcpyAsync(a->out_prob, d.out_prob, (size_t)B * 4, cudaMemcpyDeviceToHost, st));
    if (a->out_lse) CUDA_TRY(h, cudaMemcpyAsync(a->out_lse, d.out_lse, (size_t)B * 4, cudaMemcpyDeviceToHost, st));
    if (a->out_kept_ids)
        CUDA_TRY(h, cudaMemcpyAsync(a->out_kept_ids, d.out_kept_ids, (size_t)B * a->kept_stride * 4, cudaMemcpyDeviceToHost, st));
    if (a->out_kept_count)
        CUDA_TRY(h, cudaMemcpyAsync(a->out_kept_count, d.out_kept_count, (size_t)B * 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(h, cudaEventRecord(h->ev[3], st));
    CUDA_TRY(h, cudaStreamSynchronize(st));
    cudaEventElapsedTime(&h->timing[0], h->ev[0], h->ev[1]);
    cudaEventElapsedTime(&h->timing[1], h->ev[1], h->ev[2]);
    cudaEventElapsedTime(&h->timing[2], h->ev[2], h->ev[3]);
    return check_device_error(h);
}

// ---- device-resident history ------------------------------------------------------------
int32_t born_history_create(void* handle, int32_t capacity) {
    Handle* h = (Handle*)handle;
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    if (h->is_static) return fail(h, BORN_ERR_UNSUPPORTED, "the allocation-free entry point keeps no history");
    if (capacity < 1 || capacity > BORN_MAX_HISTORY) return fail(h, BORN_ERR_INVALID_ARGUMENT, "history capacity must be 1..%d", BORN_MAX_HISTORY);
    int rc = use_device(h);
    if (rc) return rc;
    cudaFree(h->ring);
    h->ring = nullptr;
    const size_t words = (size_t)h->max_batch * ((size_t)capacity + 3);
    CUDA_TRY(h, cudaMalloc((void**)&h->ring, words * 4));
    CUDA_TRY(h, cudaMemset(h->ring, 0, words * 4));
    h->ring_cap = capacity;
    h->workspace += (int64_t)words * 4;
    return BORN_OK;
}

namespace {
// ring[b][i] <- the i-th of the last min(len, cap) prompt tokens of row b; total = len = that count
__global__ void history_load_kernel(const int32_t* tokens, const int32_t* lens, int stride, int cap, int max_batch, int batch,
                                    int32_t* ring) {
    const int b = blockIdx.x;
    int32_t* meta = ring + (size_t)max_batch * cap;
    int len = lens ? lens[b] : stride;
    len = max(0, min(len, stride));
    const int keep = min(len, cap);
    for (int i = threadIdx.x; i < keep; i += blockDim.x) ring[(size_t)b * cap + i] = tokens[(size_t)b * stride + (len - keep) + i];
    if (threadIdx.x == 0) {
        meta[b] = keep;                          // total
        meta[max_batch + b] = keep;              // len
        meta[2 * (size_t)max_batch + b] = 0;     // finished
    }
    (void)batch;
}
}  // namespace

int32_t born_history_reset(void* handle, const int32_t* tokens, const int32_t* lens, int32_t batch, int32_t stride,
                           uint32_t memory, void* stream) {
    Handle* h = (Handle*)handle;
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    if (!h->ring) return fail(h, BORN_ERR_INVALID_ARGUMENT, "born_history_create has not been called");
    if (batch < 1 || batch > h->max_batch) return fail(h, BORN_ERR_INVALID_ARGUMENT, "batch %d outside 1..%d", batch, h->max_batch);
    if (stride < 0 || (stride > 0 && !tokens)) return fail(h, BORN_ERR_INVALID_ARGUMENT, "tokens is NULL with stride %d", stride);
    int rc = use_device(h);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const int32_t* d_tok = tokens;
    const int32_t* d_len = lens;
    if (memory == BORN_MEM_HOST) {
        if (stride > 0) {
            if ((rc = stage_reserve(h, 7, (size_t)batch * stride * 4))) return rc;
            CUDA_TRY(h, cudaMemcpyAsync(h->stage[7].p, tokens, (size_t)batch * stride * 4, cudaMemcpyHostToDevice, st));
            d_tok = (const int32_t*)h->stage[7].p;
        }
        if (lens) {
            if ((rc = stage_reserve(h, 8, (size_t)batch * 4))) return rc;
            CUDA_TRY(h, cudaMemcpyAsync(h->stage[8].p, lens, (size_t)batch * 4, cudaMemcpyHostToDevice, st));
            d_len = (const int32_t*)h->stage[8].p;
        }
    } else if (memory != BORN_MEM_DEVICE) {
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "memory must be BORN_MEM_DEVICE or BORN_MEM_HOST");
    }
    history_load_kernel<<<batch, 128, 0, st>>>(d_tok, d_len, stride, h->ring_cap, h->max_batch, batch, h->ring);
    CUDA_TRY(h, cudaGetLastError());
    h->launches++;
    if (memory == BORN_MEM_HOST) CUDA_TRY(h, cudaStreamSynchronize(st));  // (the caller may reuse its buffers)
    return BORN_OK;
}

int32_t born_history_set_stop_tokens(void* handle, const int32_t* ids, int32_t n) {
    Handle* h = (Handle*)handle;
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    if (n < 0 || n > 8 || (n > 0 && !ids)) return fail(h, BORN_ERR_INVALID_ARGUMENT, "0..8 stop tokens");
    h->n_stop = n;
    for (int i = 0; i < n; ++i) h->stop_ids[i] = ids[i];
    return BORN_OK;
}

int32_t born_history_read(void* handle, int32_t* tokens, int32_t* total, int32_t* finished, int32_t batch, uint32_t memory,
                          void* stream) {
    Handle* h = (Handle*)handle;
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    if (!h->ring) return fail(h, BORN_ERR_INVALID_ARGUMENT, "born_history_create has not been called");
    if (batch < 1 || batch > h->max_batch) return fail(h, BORN_ERR_INVALID_ARGUMENT, "batch %d outside 1..%d", batch, h->max_batch);
    int rc = use_device(h);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const cudaMemcpyKind kind = memory == BORN_MEM_HOST ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
    const int32_t* meta = h->ring + (size_t)h->max_batch * h->ring_cap;
    if (tokens) CUDA_TRY(h, cudaMemcpyAsync(tokens, h->ring, (size_t)batch * h->ring_cap * 4, kind, st));
    if (total) CUDA_TRY(h, cudaMemcpyAsync(total, meta, (size_t)batch * 4, kind, st));
    if (finished) CUDA_TRY(h, cudaMemcpyAsync(finished, meta + 2 * (size_t)h->max_batch, (size_t)batch * 4, kind, st));
    CUDA_TRY(h, cudaStreamSynchronize(st));
    return BORN_OK;
}

int32_t born_sample_next(void* handle, const born_sample_args* a, void* stream) {
    Handle* h = (Handle*)handle;
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    if (!h->ring) return fail(h, BORN_ERR_INVALID_ARGUMENT, "born_history_create has not been called");
    if (!a || a->struct_size != sizeof(born_sample_args)) return fail(h, BORN_ERR_INVALID_ARGUMENT, "args is NULL or of another version");
    if (a->history || a->history_len) return fail(h, BORN_ERR_INVALID_ARGUMENT, "born_sample_next reads the handle's history: args->history must be NULL");
    if (a->memory != BORN_MEM_DEVICE) return fail(h, BORN_ERR_UNSUPPORTED, "born_sample_next takes device memory");
    if (a->vocab_segments > 1) return fail(h, BORN_ERR_UNSUPPORTED, "born_sample_next does not take vocab_segments");
    born_sample_args d = *a;
    const int32_t* meta = h->ring + (size_t)h->max_batch * h->ring_cap;
    d.history = h->ring;
    d.history_len = meta + h->max_batch;
    d.history_stride = h->ring_cap;
    h->use_ring = true;
    const int32_t rc = born_sample(h, &d, stream);
    h->use_ring = false;
    return rc;
}

// ---- grammar-mask upload -----------------------------------------------------------------
int32_t born_mask_begin(void* handle, int32_t batch, int32_t words_per_row, uint32_t** host_buffer) {
    Handle* h = (Handle*)handle;
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    if (h->is_static) return fail(h, BORN_ERR_UNSUPPORTED, "the allocation-free entry point owns no mask buffers");
    if (!host_buffer || batch < 1 || words_per_row < 1) return fail(h, BORN_ERR_INVALID_ARGUMENT, "born_mask_begin: bad arguments");
    if (h->mask_filled >= 0) return fail(h, BORN_ERR_INVALID_ARGUMENT, "born_mask_begin: the previous buffer has not been committed");
    int rc = use_device(h);
    if (rc) return rc;
    const size_t words = ((size_t)batch * (size_t)words_per_row + 3) / 4 * 4;
    if (!h->mask_stream) {
        CUDA_TRY(h, cudaStreamCreateWithFlags(&h->mask_stream, cudaStreamNonBlocking));
        CUDA_TRY(h, cudaEventCreateWithFlags(&h->mask_event, cudaEventDisableTiming));
    }
    if (words > h->mask_words) {
        CUDA_TRY(h, cudaStreamSynchronize(h->mask_stream));
        CUDA_TRY(h, cudaDeviceSynchronize());  // (a kernel may still be reading the buffers about to be freed)
        for (int i = 0; i < 2; ++i) {
            if (h->mask_host[i]) cudaFreeHost(h->mask_host[i]);
            cudaFree(h->mask_dev[i]);
            h->mask_host[i] = nullptr;
            h->mask_dev[i] = nullptr;
            CUDA_TRY(h, cudaMallocHost((void**)&h->mask_host[i], words * 4));
            CUDA_TRY(h, cudaMalloc((void**)&h->mask_dev[i], words * 4));
        }
        h->mask_words = words;
    }
    // the pinned buffer may still feed the copy committed two steps ago
    CUDA_TRY(h, cudaStreamSynchronize(h->mask_stream));
    h->mask_filled = h->mask_next;
    h->mask_pending_words = words;
    *host_buffer = h->mask_host[h->mask_filled];
    return BORN_OK;
}

int32_t born_mask_commit(void* handle, const uint32_t** device_mask) {
    Handle* h = (Handle*)handle;
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    if (h->mask_filled < 0 || !device_mask) return fail(h, BORN_ERR_INVALID_ARGUMENT, "born_mask_commit without born_mask_begin");
    int rc = use_device(h);
    if (rc) return rc;
    const int i = h->mask_filled;
    CUDA_TRY(h, cudaMemcpyAsync(h->mask_dev[i], h->mask_host[i], h->mask_pending_words * 4, cudaMemcpyHostToDevice, h->mask_stream));
    CUDA_TRY(h, cudaEventRecord(h->mask_event, h->mask_stream));
    *device_mask = h->mask_dev[i];
    h->mask_filled = -1;
    h->mask_next = i ^ 1;
    return BORN_OK;
}

int32_t born_mask_wait(void* handle, void* stream) {
    Handle* h = (Handle*)handle;
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    if (!h->mask_event) return fail(h, BORN_ERR_INVALID_ARGUMENT, "born_mask_wait before any born_mask_commit");
    int rc = use_device(h);
    if (rc) return rc;
    CUDA_TRY(h, cudaStreamWaitEvent((cudaStream_t)stream, h->mask_event, 0));
    return BORN_OK;
}

int32_t born_debug_expire_wait(void* handle, void* stream) {
    Handle* h = (Handle*)handle;
    if (!h || h->is_static) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    int rc = use_device(h);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // three tiles of zeros, one row, greedy: three CTAs of one tile each; the middle one's copy is withheld
    const int V = 3 * (kTileBytes / 4);
    const size_t bytes = (size_t)V * 4 + 64;
    if ((rc = stage_reserve(h, 15, bytes))) return rc;
    uint8_t* buf = (uint8_t*)h->stage[15].p;
    CUDA_TRY(h, cudaMemsetAsync(buf, 0, bytes, st));
    ScanArgs A;
    memset(&A, 0, sizeof A);
    int grid = 0;
    if ((rc = fill_scan(h, A, 1, 1, V, BORN_DTYPE_F32, buf, V, nullptr, 0, &grid))) return rc;
    A.params.flags = BORN_FLAG_GREEDY;
    A.out_token = (int32_t*)(buf + (size_t)V * 4);
    A.out_status = (int32_t*)(buf + (size_t)V * 4 + 16);
    A.mode = kScanFull;
    A.timeout_ns = 1000000ull;
    A.debug_skip_tile = 1;
    if ((rc = launch_scan(h, A, BORN_DTYPE_F32, grid, st))) return rc;
    CUDA_TRY(h, cudaStreamSynchronize(st));
    return check_device_error(h);
}

int32_t born_debug_exp(const float* x, float* y, int64_t n, void* stream) {
    if (!x || !y || n < 0) return BORN_ERR_INVALID_ARGUMENT;
    if (n == 0) return BORN_OK;
    debug_exp_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, y, n);
    return cudaGetLastError() == cudaSuccess ? BORN_OK : BORN_ERR_CUDA;
}
int32_t born_debug_mass(const float* x, uint64_t* q, int64_t n, void* stream) {
    if (!x || !q || n < 0) return BORN_ERR_INVALID_ARGUMENT;
    if (n == 0) return BORN_OK;
    debug_mass_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, (unsigned long long*)q, n);
    return cudaGetLastError() == cudaSuccess ? BORN_OK : BORN_ERR_CUDA;
}

// ------------------------------------------------------------------ speculative verify
int32_t born_spec_verify(void* handle, const born_spec_args* a, void* stream) {
    Handle* h = (Handle*)handle;
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    if (!a || a->struct_size != sizeof(born_spec_args)) return fail(h, BORN_ERR_INVALID_ARGUMENT, "args NULL or wrong struct_size");
    const int B = a->batch, K = a->draft_len, V = a->vocab, R = a->target_rows;
    if (B <= 0 || K <= 0 || V <= 0 || K > BORN_MAX_DRAFT || (R != K && R != K + 1))
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "spec_verify: batch=%d draft_len=%d vocab=%d target_rows=%d", B, K, V, R);
    if (B > h->max_batch || V > h->max_vocab) return fail(h, BORN_ERR_INVALID_ARGUMENT, "batch/vocab exceed the handle");
    if (!a->target_logits || !a->draft_logits || !a->draft_tokens || !a->u_accept || !a->u_resample ||
        !a->out_accept_len || !a->out_tokens || !a->out_status)
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "spec_verify: a required pointer is NULL");
    if (!(a->temperature >= 0.0f) || !isfinite(a->temperature)) return fail(h, BORN_ERR_INVALID_ARGUMENT, "temperature");
    if (V > kSpecMaxBlocks * kSpecMassBlock)
        return fail(h, BORN_ERR_UNSUPPORTED, "spec_verify: vocab %d exceeds %d", V, kSpecMaxBlocks * kSpecMassBlock);
    if (a->memory != BORN_MEM_DEVICE && a->memory != BORN_MEM_HOST) return fail(h, BORN_ERR_INVALID_ARGUMENT, "memory");
    { int rcd = use_device(h); if (rcd) return rcd; }
    cudaStream_t st = (cudaStream_t)stream;
    SpecKernelArgs A;
    memset(&A, 0, sizeof A);
    A.B = B; A.K = K; A.V = V; A.target_rows = R;
    A.inv_T = a->temperature == 0.0f ? 1.0f : 1.0f / a->temperature;
    // scratch of the speculative path (tickets, chunk sums, block results): grown on first use
    // like the staging mirrors, then reused; the tickets are zero between launches
    const SpecScratchLayout SL = spec_scratch_layout(B, K, V);
    if (h->spec_scratch_bytes < SL.total) {
        int rc0 = grow(h, (void**)&h->spec_scratch, &h->spec_scratch_bytes, SL.total, st);
        if (rc0 != BORN_OK) return rc0;
        h->spec_layout_key = -1;
    }
    // the ticket area sits at offset 0 whatever the shape; it is cleared when the layout changes
    if (h->spec_layout_key != ((int64_t)B << 40 | (int64_t)K << 32 | (int64_t)V)) {
        CUDA_TRY(h, cudaMemsetAsync(h->spec_scratch, 0, SL.csum, st));
        h->spec_layout_key = ((int64_t)B << 40 | (int64_t)K << 32 | (int64_t)V);
    }
    A.tickets = reinterpret_cast<uint32_t*>(h->spec_scratch + SL.tickets);
    A.csum = reinterpret_cast<unsigned long long*>(h->spec_scratch + SL.csum);
    A.blocks = reinterpret_cast<BlockMass*>(h->spec_scratch + SL.blocks);
    A.dev_error = h->dev_error;
    if (a->memory == BORN_MEM_DEVICE) {
        A.target = a->target_logits; A.draft = a->draft_logits; A.draft_tok = a->draft_tokens;
        A.u_accept = a->u_accept; A.u_resample = a->u_resample;
        A.accept_len = a->out_accept_len; A.out_tok = a->out_tokens; A.status = a->out_status;
        int rc = launch_spec(A, h->num_sms, st);
        if (rc != 0) return fail(h, BORN_ERR_CUDA, "spec kernel launch failed: %s", cudaGetErrorString((cudaError_t)rc));
        h->launches += 2;
        return BORN_OK;
    }
    if (a->memory != BORN_MEM_HOST) return fail(h, BORN_ERR_INVALID_ARGUMENT, "memory");
    int rc;
    const size_t nt = (size_t)B * R * V * 4, nd = (size_t)B * K * V * 4;
    if ((rc = stage_reserve(h, 0, nt))) return rc;
    if ((rc = stage_reserve(h, 1, nd))) return rc;
    if ((rc = stage_reserve(h, 2, (size_t)B * K * 4))) return rc;
    if ((rc = stage_reserve(h, 3, (size_t)B * K * 4))) return rc;
    if ((rc = stage_reserve(h, 4, (size_t)B * (K + 1) * 4))) return rc;
    if ((rc = stage_reserve(h, 6, (size_t)B * 4))) return rc;
    if ((rc = stage_reserve(h, 7, (size_t)B * (K + 1) * 4))) return rc;
    if ((rc = stage_reserve(h, 9, (size_t)B * 4))) return rc;
    CUDA_TRY(h, cudaEventRecord(h->ev[0], st));
    CUDA_TRY(h, cudaMemcpyAsync(h->stage[0].p, a->target_logits, nt, cudaMemcpyHostToDevice, st));
    CUDA_TRY(h, cudaMemcpyAsync(h->stage[1].p, a->draft_logits, nd, cudaMemcpyHostToDevice, st));
    CUDA_TRY(h, cudaMemcpyAsync(h->stage[2].p, a->draft_tokens, (size_t)B * K * 4, cudaMemcpyHostToDevice, st));
    CUDA_TRY(h, cudaMemcpyAsync(h->stage[3].p, a->u_accept, (size_t)B * K * 4, cudaMemcpyHostToDevice, st));
    CUDA_TRY(h, cudaMemcpyAsync(h->stage[4].p, a->u_resample, (size_t)B * (K + 1) * 4, cudaMemcpyHostToDevice, st));
    A.target = (const float*)h->stage[0].p; A.draft = (const float*)h->stage[1].p;
    A.draft_tok = (const int32_t*)h->stage[2].p; A.u_accept = (const float*)h->stage[3].p;
    A.u_resample = (const float*)h->stage[4].p;
    A.accept_len = (int32_t*)h->stage[6].p; A.out_tok = (int32_t*)h->stage[7].p; A.status = (int32_t*)h->stage[9].p;
    CUDA_TRY(h, cudaEventRecord(h->ev[1], st));
    rc = launch_spec(A, h->num_sms, st);
    if (rc != 0) return fail(h, BORN_ERR_CUDA, "spec kernel launch failed: %s", cudaGetErrorString((cudaError_t)rc));
    h->launches += 2;
    CUDA_TRY(h, cudaEventRecord(h->ev[2], st));
    CUDA_TRY(h, cudaMemcpyAsync(a->out_accept_len, A.accept_len, (size_t)B * 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(h, cudaMemcpyAsync(a->out_tokens, A.out_tok, (size_t)B * (K + 1) * 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(h, cudaMemcpyAsync(a->out_status, A.status, (size_t)B * 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(h, cudaEventRecord(h->ev[3], st));
    CUDA_TRY(h, cudaStreamSynchronize(st));
    cudaEventElapsedTime(&h->timing[0], h->ev[0], h->ev[1]);
    cudaEventElapsedTime(&h->timing[1], h->ev[1], h->ev[2]);
    cudaEventElapsedTime(&h->timing[2], h->ev[2], h->ev[3]);
    return check_device_error(h);
}

// ------------------------------------------------------------------ vocab-sharded path
int32_t born_shard_record_bytes(int32_t top_k) {
    if (top_k <= 0 || top_k > BORN_MAX_TOP_K) return -1;
    return kRecordHdrBytes + 8 * top_k;
}

static int nccl_load(Handle* h) {
    if (h->nccl.lib) return BORN_OK;
    void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) return fail(h, BORN_ERR_NCCL, "cannot load libnccl.so.2: %s", dlerror());
    NcclApi& n = h->nccl;
    n.GetUniqueId = (int (*)(void*))dlsym(lib, "ncclGetUniqueId");
    n.CommInitRank = (int (*)(void**, int, Id128, int))dlsym(lib, "ncclCommInitRank");
    n.AllGather = (int (*)(const void*, void*, size_t, int, void*, cudaStream_t))dlsym(lib, "ncclAllGather");
    n.CommDestroy = (int (*)(void*))dlsym(lib, "ncclCommDestroy");
    n.GetErrorString = (const char* (*)(int))dlsym(lib, "ncclGetErrorString");
    if (!n.GetUniqueId || !n.CommInitRank || !n.AllGather || !n.CommDestroy)
        return fail(h, BORN_ERR_NCCL, "libnccl.so.2 lacks a required symbol");
    n.lib = lib;
    return BORN_OK;
}

int32_t born_shard_unique_id(void* out_id128) {
    if (!out_id128) return BORN_ERR_INVALID_ARGUMENT;
    Handle tmp;
    int rc = nccl_load(&tmp);
    if (rc) { snprintf(g_err, sizeof g_err, "%s", tmp.err); return rc; }
    int e = tmp.nccl.GetUniqueId(out_id128);
    return e == 0 ? BORN_OK : BORN_ERR_NCCL;
}

int32_t born_shard_init(void* handle, const void* id, int32_t rank, int32_t nranks) {
    Handle* h = (Handle*)handle;
    if (!h || !id) return fail(h, BORN_ERR_INVALID_ARGUMENT, "shard_init: NULL argument");
    if (nranks < 1 || nranks > BORN_MAX_SHARDS || rank < 0 || rank >= nranks)
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "shard_init: rank %d of %d", rank, nranks);
    int rc = nccl_load(h);
    if (rc) return rc;
    { int rcd = use_device(h); if (rcd) return rcd; }
    Id128 u;
    memcpy(&u, id, sizeof u);
    int e = h->nccl.CommInitRank(&h->comm, nranks, u, rank);
    if (e != 0) return fail(h, BORN_ERR_NCCL, "ncclCommInitRank: %s", h->nccl.GetErrorString ? h->nccl.GetErrorString(e) : "error");
    h->rank = rank;
    h->nranks = nranks;
    // exchange buffers for the handle's limits (top_k <= 256 per shard): nothing is allocated per call
    const size_t pk = (size_t)h->max_batch * (size_t)(kRecordHdrBytes + 8 * kThreads);
    if ((rc = grow(h, (void**)&h->packed, &h->packed_bytes, pk, nullptr))) return rc;
    if ((rc = grow(h, (void**)&h->gathered, &h->gathered_bytes, pk * (size_t)nranks, nullptr))) return rc;
    return BORN_OK;
}

static int shard_check(Handle* h, const born_shard_args* a, bool local, bool merge) {
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    if (!a || a->struct_size != sizeof(born_shard_args)) return fail(h, BORN_ERR_INVALID_ARGUMENT, "args NULL or wrong struct_size");
    if (a->memory != BORN_MEM_DEVICE) return fail(h, BORN_ERR_UNSUPPORTED, "the sharded path takes device memory only");
    if (a->batch <= 0 || a->batch > h->max_rows || a->vocab_local <= 0 || a->vocab_local > h->max_vocab)
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "batch/vocab_local out of range");
    if (a->nranks < 1 || a->nranks > BORN_MAX_SHARDS || a->rank < 0 || a->rank >= a->nranks)
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "rank %d of %d", a->rank, a->nranks);
    if ((int64_t)a->vocab_local * a->nranks > BORN_MAX_VOCAB) return fail(h, BORN_ERR_UNSUPPORTED, "global vocab too large");
    if (a->top_k <= 0 || (int64_t)a->top_k * a->nranks > BORN_MAX_CANDIDATES)
        return fail(h, BORN_ERR_UNSUPPORTED, "need 1 <= top_k*nranks <= %d", BORN_MAX_CANDIDATES);
    if (a->top_k > kThreads) return fail(h, BORN_ERR_UNSUPPORTED, "the sharded path takes top_k <= %d per shard", kThreads);
    if (!(a->temperature > 0.0f) || !isfinite(a->temperature) || !(a->top_p >= 0.0f))
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "temperature must be > 0 and top_p >= 0");
    if (local) {
        if (!a->logits || a->logits_row_stride < a->vocab_local) return fail(h, BORN_ERR_INVALID_ARGUMENT, "logits");
        if (a->logits_dtype != BORN_DTYPE_F32 && a->logits_dtype != BORN_DTYPE_BF16) return fail(h, BORN_ERR_INVALID_ARGUMENT, "dtype");
    }
    if (merge && (!a->uniforms || !a->out_token || !a->out_status)) return fail(h, BORN_ERR_INVALID_ARGUMENT, "uniforms/out_token/out_status");
    return BORN_OK;
}

// Local pass of one shard: the k best of every row (global token ids), the shard's maximum
// and its share of the log-sum-exp, one packed record per row.
static int shard_local(Handle* h, const born_shard_args* a, void* packed, bool want_lse, cudaStream_t st) {
    ScanArgs A;
    memset(&A, 0, sizeof A);
    int grid = 0;
    int rc = fill_scan(h, A, a->batch, 1, a->vocab_local, a->logits_dtype, a->logits, a->logits_row_stride, nullptr, 0, &grid);
    if (rc) return rc;
    A.params.temperature = a->temperature;
    A.params.top_p = a->top_p;
    A.params.top_k = a->top_k;
    A.params.repetition_penalty = 1.0f;
    A.mode = kScanLocal;
    A.want_lse = want_lse ? 1 : 0;
    A.idx_base = a->rank * a->vocab_local;
    A.packed = (uint8_t*)packed;
    A.packed_row_stride = born_shard_record_bytes(a->top_k);
    A.packed_seg_stride = 0;
    return launch_scan(h, A, a->logits_dtype, grid, st);
}

static int shard_merge(Handle* h, const born_shard_args* a, const void* gathered, cudaStream_t st) {
    MergeArgs M;
    memset(&M, 0, sizeof M);
    M.gathered = (const uint8_t*)gathered;
    M.row_stride = born_shard_record_bytes(a->top_k);
    M.seg_stride = M.row_stride * a->batch;
    M.B = a->batch; M.G = a->nranks;
    M.temperature = a->temperature; M.top_p = a->top_p;
    M.uniforms = a->uniforms;
    M.out_token = a->out_token; M.out_prob = a->out_prob; M.out_lse = a->out_lse; M.out_status = a->out_status;
    return launch_merge(h, M, st);
}

int32_t born_shard_local(void* handle, const born_shard_args* a, void* stream) {
    Handle* h = (Handle*)handle;
    int rc = shard_check(h, a, true, false);
    if (rc) return rc;
    if (!a->packed) return fail(h, BORN_ERR_INVALID_ARGUMENT, "packed is NULL");
    if ((rc = use_device(h))) return rc;
    return shard_local(h, a, a->packed, true, (cudaStream_t)stream);
}

int32_t born_shard_merge(void* handle, const born_shard_args* a, void* stream) {
    Handle* h = (Handle*)handle;
    int rc = shard_check(h, a, false, true);
    if (rc) return rc;
    if (!a->gathered) return fail(h, BORN_ERR_INVALID_ARGUMENT, "gathered is NULL");
    if ((rc = use_device(h))) return rc;
    return shard_merge(h, a, a->gathered, (cudaStream_t)stream);
}

int32_t born_sample_sharded(void* handle, const born_shard_args* a, void* stream) {
    Handle* h = (Handle*)handle;
    int rc = shard_check(h, a, true, true);
    if (rc) return rc;
    if (!h->comm) return fail(h, BORN_ERR_NCCL, "born_shard_init has not been called on this handle");
    if (a->nranks != h->nranks || a->rank != h->rank) return fail(h, BORN_ERR_INVALID_ARGUMENT, "rank/nranks differ from born_shard_init");
    if ((rc = use_device(h))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t rec = (size_t)born_shard_record_bytes(a->top_k);
    const size_t pk = rec * (size_t)a->batch, ga = pk * (size_t)a->nranks;
    // exchange buffers: sized by born_shard_init for the handle's limits, grown here only by a larger request
    if ((rc = grow(h, (void**)&h->packed, &h->packed_bytes, pk, st))) return rc;
    if ((rc = grow(h, (void**)&h->gathered, &h->gathered_bytes, ga, st))) return rc;
    if ((rc = shard_local(h, a, h->packed, a->out_lse != nullptr, st))) return rc;
    int e = h->nccl.AllGather(h->packed, h->gathered, pk, /*ncclInt8*/ 0, h->comm, st);
    if (e != 0) return fail(h, BORN_ERR_NCCL, "ncclAllGather: %s", h->nccl.GetErrorString ? h->nccl.GetErrorString(e) : "error");
    return shard_merge(h, a, h->gathered, st);
}

}  // extern "C"

// ------------------------------------------------------------------ allocation-free entry
// Scratch for born_sample_static: segment records, mass blocks, row tickets and the device
// error word in one file-scope array that every GPU loading this library holds until exit.
namespace {
constexpr int kStaticMaxBatch = BORN_STATIC_MAX_BATCH;
constexpr int kStaticRecCap = 512;
constexpr int kStaticMaxGrid = 512;  // >= two CTAs per SM on any sm_100 part
constexpr size_t kStaticRecStride = kRecordHdrBytes + (size_t)kStaticRecCap * 8;
constexpr size_t kStaticRecordsBytes = (size_t)(kStaticMaxBatch + kStaticMaxGrid) * kStaticRecStride;
constexpr size_t kStaticBlocks = BORN_STATIC_MAX_BLOCKS;
constexpr size_t kStaticBlocksBytes = kStaticBlocks * sizeof(MassBlock);
constexpr size_t kStaticTicketsBytes = sizeof(uint32_t) * 2 * kStaticMaxBatch;
constexpr size_t kStaticBytes = kStaticRecordsBytes + kStaticBlocksBytes + kStaticTicketsBytes + 256;  // (the last 256: error word and counters)
static_assert(kStaticBytes <= BORN_STATIC_SCRATCH_BYTES, "the header promises at most BORN_STATIC_SCRATCH_BYTES");
constexpr int kStaticMaxDevices = 64;
}  // namespace

static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

namespace {
Handle g_static_handle[kStaticMaxDevices];
bool g_static_ready[kStaticMaxDevices];
}  // namespace

extern "C" int32_t born_sample_static(const born_sample_args* a, void* stream) {
    if (!a) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "born_sample_static: args is NULL");
    if (a->struct_size != sizeof(born_sample_args))
        return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "born_sample_static: struct_size %u != %zu", a->struct_size,
                    sizeof(born_sample_args));
    if (a->memory != BORN_MEM_DEVICE)
        return fail(nullptr, BORN_ERR_UNSUPPORTED,
                    "born_sample_static takes device memory only (a host-memory call would need staging buffers)");
    if (a->batch > kStaticMaxBatch)
        return fail(nullptr, BORN_ERR_UNSUPPORTED, "born_sample_static: batch %d exceeds the static scratch limit of %d rows",
                    a->batch, kStaticMaxBatch);
    if (a->batch > 0 && a->vocab > 0 &&
        (int64_t)a->batch * (((int64_t)a->vocab + kMassBlock - 1) / kMassBlock) > (int64_t)kStaticBlocks)
        return fail(nullptr, BORN_ERR_UNSUPPORTED, "born_sample_static: batch x ceil(vocab/%d) exceeds %d mass blocks of static scratch",
                    kMassBlock, (int)kStaticBlocks);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(nullptr, BORN_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kStaticMaxDevices) return fail(nullptr, BORN_ERR_UNSUPPORTED, "device index %d not supported", dev);
    Handle* h = &g_static_handle[dev];
    if (!g_static_ready[dev]) {
        // First call on this device (it is the current one): turn the symbol into a device
        // address.  In host code the array's name is only a stand-in, not a device pointer.
        unsigned char* base = nullptr;
        e = cudaGetSymbolAddress((void**)&base, g_static_scratch);
        if (e != cudaSuccess || !base)
            return fail(nullptr, BORN_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        int sms = 0, major = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
            return fail(nullptr, BORN_ERR_CUDA, "cudaDeviceGetAttribute failed");
        if (major != 10) return fail(nullptr, BORN_ERR_NO_DEVICE, "device %d is not sm_100; this library is built for sm_100a only", dev);
        if ((e = scan_attrs_all()) != cudaSuccess)
            return fail(nullptr, BORN_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
        h->device = dev;
        h->is_static = true;
        h->max_batch = kStaticMaxBatch;
        h->max_vocab = BORN_MAX_VOCAB;
        h->max_k = BORN_MAX_TOP_K;
        h->num_sms = sms;
        h->max_grid = 2 * sms < kStaticMaxGrid ? 2 * sms : kStaticMaxGrid;
        h->max_rows = kStaticMaxBatch;
        h->rec_cap = kStaticRecCap;
        h->rec_stride = (int64_t)kStaticRecStride;
        h->records_bytes = kStaticRecordsBytes;
        h->records = base;
        h->blocks = reinterpret_cast<MassBlock*>(base + kStaticRecordsBytes);
        h->blocks_cap = (int64_t)kStaticBlocks;
        h->tickets = reinterpret_cast<uint32_t*>(base + kStaticRecordsBytes + kStaticBlocksBytes);
        h->dev_error = reinterpret_cast<int*>(base + kStaticRecordsBytes + kStaticBlocksBytes + kStaticTicketsBytes);
        g_static_ready[dev] = true;
    }
    // The array keeps whatever the previous call left; the tickets and the error word
    // must start at zero.
    e = cudaMemsetAsync(h->tickets, 0, kStaticTicketsBytes + 256, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(nullptr, BORN_ERR_CUDA, "cudaMemsetAsync(static scratch) failed: %s", cudaGetErrorString(e));
    int32_t rc = born_sample(h, a, stream);
    if (rc != BORN_OK) snprintf(g_err, sizeof g_err, "%.500s", h->err);
    return rc;
}
