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
#include "sample_kernel.cuh"
#include "spec_kernel.cuh"
#include "fullrow_kernel.cuh"

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
    int max_records = 0;
    int64_t record_stride = 0;
    uint8_t* records = nullptr;
    uint32_t* tickets = nullptr;
    int* dev_error = nullptr;
    uint8_t* spec_scratch = nullptr;
    size_t spec_scratch_bytes = 0;
    int64_t spec_layout_key = -1;
    uint8_t* fr_scratch = nullptr;  // full-vocabulary path: tickets, range statistics, chunk sums
    size_t fr_scratch_bytes = 0;
    int64_t fr_layout_key = -1;
    bool is_static = false;  // the handle of born_sample_static: may not allocate
    float* pen_copy = nullptr;  // fp32 copy of the rows with history penalties applied (whole-vocabulary routes)
    size_t pen_copy_bytes = 0;
    Staging stage[16];
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
    float timing[3] = {0, 0, 0};
    int64_t launches = 0;
    int64_t workspace = 0;
    int force_slices = 0;
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
    cudaError_t e = cudaMalloc(p, bytes);
    if (e != cudaSuccess) return fail(h, BORN_ERR_CUDA, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    h->workspace += (int64_t)bytes;
    return BORN_OK;
}

int stage_reserve(Handle* h, int slot, size_t bytes) {
    Staging& s = h->stage[slot];
    if (s.bytes >= bytes) return BORN_OK;
    if (s.p) { cudaFree(s.p); h->workspace -= (int64_t)s.bytes; s.p = nullptr; s.bytes = 0; }
    int rc = dev_alloc(h, &s.p, bytes);
    if (rc == BORN_OK) s.bytes = bytes;
    return rc;
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

template <typename T, bool M, bool Lse>
int launch_variant(Handle* h, const SampleKernelArgs& A, dim3 grid, size_t smem, cudaStream_t st) {
    auto kern = sample_kernel<T, M, Lse>;
    CUDA_TRY(h, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kBlockThreads, smem, st>>>(A);
    CUDA_TRY(h, cudaGetLastError());
    h->launches++;
    return BORN_OK;
}

int launch_sample(Handle* h, const SampleKernelArgs& A, int dtype, cudaStream_t st) {
    const bool has_mask = A.mask != nullptr, lse = A.out_lse != nullptr;
    const SmemLayout L = smem_layout(dtype == BORN_DTYPE_F32 ? 4 : 2, has_mask, A.history != nullptr);
    dim3 grid((unsigned)(A.mode == kModeMerge ? 1 : A.S), (unsigned)A.B, 1);
    const size_t smem = (size_t)L.total;
#define V_(T, M, Lq) return launch_variant<T, M, Lq>(h, A, grid, smem, st)
    if (dtype == BORN_DTYPE_F32) {
        if (has_mask) { if (lse) V_(float, true, true); else V_(float, true, false); }
        else { if (lse) V_(float, false, true); else V_(float, false, false); }
    } else {
        if (has_mask) { if (lse) V_(uint16_t, true, true); else V_(uint16_t, true, false); }
        else { if (lse) V_(uint16_t, false, true); else V_(uint16_t, false, false); }
    }
#undef V_
}

// Slices per row.  With at least one row per SM every row is one CTA (a slice costs a
// threshold bootstrap and a record merge); smaller batches are cut so that about two CTAs
// per SM exist, but never below four tiles per slice.
void choose_slices(const Handle* h, int B, int V, int elem_bytes, int* S, int* slice_len) {
    const int kChunk = kTileBytes / elem_bytes;  // logits per pipeline stage
    const int nchunks = (V + kChunk - 1) / kChunk;
    int s = 1;
    if (h->force_slices > 0) s = h->force_slices;
    else if (B < h->num_sms) {
        s = (2 * h->num_sms + B - 1) / B;
        int cap = nchunks / 4;
        if (cap < 1) cap = 1;
        if (s > cap) s = cap;
    }
    if (s > 64) s = 64;
    if (s > nchunks) s = nchunks;
    while (s > 1 && (int64_t)s * B > h->max_records) --s;
    if (s < 1) s = 1;
    int per = (nchunks + s - 1) / s;
    *slice_len = per * kChunk;
    *S = (nchunks + per - 1) / per;
}

int check_device_error(Handle* h) {
    int e = 0;
    CUDA_TRY(h, cudaMemcpy(&e, h->dev_error, sizeof(int), cudaMemcpyDeviceToHost));
    if (e) {
        cudaMemset(h->dev_error, 0, sizeof(int));
        return fail(h, BORN_ERR_DEVICE_TIMEOUT, "a bounded on-device wait gave up (code %d); outputs are invalid", e);
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

}  // namespace

extern "C" {

const char* born_version(void) { return "born-sampler-b200 0.1.0 (sm_100a)"; }

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
    h->max_k = max_k;
    h->num_sms = prop.multiProcessorCount;
    const char* fs = getenv("BORN_SLICES");
    if (fs) h->force_slices = atoi(fs);
    if (cudaSetDevice(device) != cudaSuccess) { delete h; return fail(nullptr, BORN_ERR_CUDA, "cudaSetDevice failed"); }
    h->max_records = max_batch * 4 > 2048 ? max_batch * 4 : 2048;
    h->record_stride = kRecordHdrBytes + (int64_t)kMaxK * 8;
    int rc = dev_alloc(h, (void**)&h->records, (size_t)h->max_records * (size_t)h->record_stride);
    if (rc == BORN_OK) rc = dev_alloc(h, (void**)&h->tickets, sizeof(uint32_t) * (size_t)max_batch * 2);
    if (rc == BORN_OK) rc = dev_alloc(h, (void**)&h->dev_error, sizeof(int));
    if (rc == BORN_OK && cudaMemset(h->tickets, 0, sizeof(uint32_t) * (size_t)max_batch * 2) != cudaSuccess) rc = BORN_ERR_CUDA;
    if (rc == BORN_OK && cudaMemset(h->dev_error, 0, sizeof(int)) != cudaSuccess) rc = BORN_ERR_CUDA;
    for (int i = 0; i < 4 && rc == BORN_OK; ++i)
        if (cudaEventCreate(&h->ev[i]) != cudaSuccess) rc = BORN_ERR_CUDA;
    if (rc != BORN_OK) {
        snprintf(g_err, sizeof g_err, "create failed: %.480s", h->err[0] ? h->err : "CUDA error");
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
    cudaFree(h->records);
    cudaFree(h->tickets);
    cudaFree(h->dev_error);
    cudaFree(h->spec_scratch);
    cudaFree(h->fr_scratch);
    cudaFree(h->pen_copy);
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

// Rows that neither top-k nor top-p narrows have no small candidate set: temperature-only
// sampling always, min-p when the caller asks for it with BORN_FLAG_FULL_VOCAB (without the
// flag min-p goes through the one-pass kernel, which serves up to 1024 survivors).  Uniform
// parameters only, no history penalties, no kept-id list.
static bool wants_full_row(const Handle* h, const born_sample_args* a) {
    if (h->is_static || a->row_params || a->vocab_segments > 1 || a->out_kept_ids) return false;
    const born_row_params& p = a->params;
    if ((p.flags & BORN_FLAG_GREEDY) || p.temperature == 0.0f) return false;
    if (p.top_k > 0 || (p.top_p > 0.0f && p.top_p < 1.0f)) return false;
    if (p.min_p > 0.0f && !(p.flags & BORN_FLAG_FULL_VOCAB)) return false;
    const bool pen_on = (p.repetition_penalty != 1.0f && p.repetition_penalty != 0.0f) || p.frequency_penalty != 0.0f ||
                        p.presence_penalty != 0.0f;
    if (a->history && pen_on) return false;
    return true;
}

// Top-p without top-k: the one-pass kernel keeps the 1024 best, which hold the nucleus of any
// peaked distribution, but the nucleus is defined against the total mass of all survivors.
// That total comes from the two passes of the whole-vocabulary path (run in sum-only mode).
static bool wants_survivor_total(const Handle* h, const born_sample_args* a) {
    if (h->is_static || a->row_params || a->vocab_segments > 1) return false;
    const born_row_params& p = a->params;
    if ((p.flags & BORN_FLAG_GREEDY) || p.temperature == 0.0f) return false;
    if (p.top_k > 0 || !(p.top_p > 0.0f && p.top_p < 1.0f)) return false;
    // min-p already narrows the row for the one-pass kernel (up to 1024 survivors): the extra
    // passes are only taken when the caller asks for them
    if (p.min_p > 0.0f && !(p.flags & BORN_FLAG_FULL_VOCAB)) return false;
    const bool pen_on = (p.repetition_penalty != 1.0f && p.repetition_penalty != 0.0f) || p.frequency_penalty != 0.0f ||
                        p.presence_penalty != 0.0f;
    if (a->history && pen_on) return false;
    return true;
}

// Both launches of the whole-vocabulary path; with `totals_only` the second one leaves each row's
// total survivor mass in *totals and writes no outputs.
static int run_full_row(Handle* h, const born_sample_args* a, cudaStream_t st, bool totals_only,
                        const unsigned long long** totals) {
    const int B = a->batch, V = a->vocab;
    const int esz = a->logits_dtype == BORN_DTYPE_F32 ? 4 : 2;
    const int parts = fullrow_parts(B, V, h->num_sms);
    const FullRowScratchLayout L = fullrow_scratch_layout(B, V, parts);
    if (h->fr_scratch_bytes < L.total) {  // grown on first use, like the staging mirrors
        CUDA_TRY(h, cudaStreamSynchronize(st));
        if (h->fr_scratch) { cudaFree(h->fr_scratch); h->workspace -= (int64_t)h->fr_scratch_bytes; h->fr_scratch = nullptr; h->fr_scratch_bytes = 0; }
        int rc0 = dev_alloc(h, (void**)&h->fr_scratch, L.total);
        if (rc0 != BORN_OK) return rc0;
        h->fr_scratch_bytes = L.total;
        h->fr_layout_key = -1;
    }
    const int64_t key = ((int64_t)B << 32) | (int64_t)V;
    if (h->fr_layout_key != key) {  // the tickets sit at offset 0 and are zero between launches
        CUDA_TRY(h, cudaMemsetAsync(h->fr_scratch, 0, L.stat, st));
        h->fr_layout_key = key;
    }
    FullRowArgs F;
    memset(&F, 0, sizeof F);
    F.logits = a->logits;
    F.mask = a->mask;
    F.uniforms = a->uniforms;
    F.out_token = a->out_token; F.out_prob = a->out_prob; F.out_lse = a->out_lse; F.out_status = a->out_status;
    F.out_kept_count = a->out_kept_count;
    F.tickets = reinterpret_cast<uint32_t*>(h->fr_scratch + L.tickets);
    F.stat = reinterpret_cast<float2*>(h->fr_scratch + L.stat);
    F.csum = reinterpret_cast<unsigned long long*>(h->fr_scratch + L.csum);
    F.ccount = reinterpret_cast<uint32_t*>(h->fr_scratch + L.ccount);
    F.total_out = totals_only ? reinterpret_cast<unsigned long long*>(h->fr_scratch + L.totals) : nullptr;
    if (totals_only) F.out_kept_count = nullptr;
    F.row_stride = a->logits_row_stride;
    F.mask_stride = a->mask_row_stride;
    F.B = B; F.V = V; F.parts1 = parts;
    F.temperature = a->params.temperature;
    F.min_p = a->params.min_p;
    F.vec_ok = ((uintptr_t)a->logits % 16 == 0) && ((a->logits_row_stride * esz) % 16 == 0);
    int rc = launch_fullrow(F, a->logits_dtype, parts, st);
    if (rc != 0) return fail(h, BORN_ERR_CUDA, "full-vocabulary kernel launch failed: %s", cudaGetErrorString((cudaError_t)rc));
    h->launches += 2;
    if (totals) *totals = F.total_out;
    return BORN_OK;
}

static int sample_full_row(Handle* h, const born_sample_args* a, cudaStream_t st) {
    return run_full_row(h, a, st, false, nullptr);
}

static int sample_device(Handle* h, const born_sample_args* a_in, cudaStream_t st) {
    const born_sample_args* a = a_in;
    born_sample_args a2;
    {
        // The whole-vocabulary routes read the raw logits more than once.  A row with history
        // penalties that would take one of them is first copied, penalties applied, to fp32
        // scratch; the routes then see plain rows without a history.
        const born_row_params& p = a_in->params;
        const bool pen_on = (p.repetition_penalty != 1.0f && p.repetition_penalty != 0.0f) || p.frequency_penalty != 0.0f ||
                            p.presence_penalty != 0.0f;
        if (a_in->history && pen_on && !a_in->row_params) {
            a2 = *a_in;
            a2.history = nullptr; a2.history_len = nullptr; a2.history_stride = 0;
            a2.params.repetition_penalty = 0.0f; a2.params.frequency_penalty = 0.0f; a2.params.presence_penalty = 0.0f;
            if (wants_full_row(h, &a2) || wants_survivor_total(h, &a2)) {
                const int64_t v_pad = ((int64_t)a_in->vocab + 3) / 4 * 4;
                const size_t need = (size_t)a_in->batch * (size_t)v_pad * sizeof(float);
                if (h->pen_copy_bytes < need) {  // grown on first use, like the staging mirrors
                    CUDA_TRY(h, cudaStreamSynchronize(st));
                    if (h->pen_copy) { cudaFree(h->pen_copy); h->workspace -= (int64_t)h->pen_copy_bytes; h->pen_copy = nullptr; h->pen_copy_bytes = 0; }
                    int rc0 = dev_alloc(h, (void**)&h->pen_copy, need);
                    if (rc0 != BORN_OK) return rc0;
                    h->pen_copy_bytes = need;
                }
                PenaliseArgs P;
                memset(&P, 0, sizeof P);
                P.logits = a_in->logits; P.out = h->pen_copy;
                P.history = a_in->history; P.history_len = a_in->history_len;
                P.row_stride = a_in->logits_row_stride; P.out_stride = v_pad;
                P.B = a_in->batch; P.V = a_in->vocab; P.history_stride = a_in->history_stride;
                P.repetition = p.repetition_penalty; P.frequency = p.frequency_penalty; P.presence = p.presence_penalty;
                int rc1 = launch_penalised_copy(P, a_in->logits_dtype, h->num_sms, st);
                if (rc1 != 0) return fail(h, BORN_ERR_CUDA, "penalised-copy launch failed: %s", cudaGetErrorString((cudaError_t)rc1));
                h->launches += 2;
                a2.logits = h->pen_copy;
                a2.logits_dtype = BORN_DTYPE_F32;
                a2.logits_row_stride = v_pad;
                a = &a2;
            }
        }
    }
    if (wants_full_row(h, a)) return sample_full_row(h, a, st);
    const unsigned long long* survivor_total = nullptr;
    if (wants_survivor_total(h, a)) {
        int rc0 = run_full_row(h, a, st, true, &survivor_total);
        if (rc0 != BORN_OK) return rc0;
    }
    SampleKernelArgs A;
    memset(&A, 0, sizeof A);
    A.ext_total = survivor_total;
    A.logits = a->logits;
    A.row_stride = a->logits_row_stride;
    A.mask = a->mask;
    A.mask_stride = a->mask_row_stride;
    A.history = a->history;
    A.history_len = a->history_len;
    A.history_stride = a->history_stride;
    A.B = a->batch;
    A.V = a->vocab;
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
    A.mode = kModeFull;
    A.records = h->records;
    A.rec_slice_stride = h->record_stride;
    A.tickets = h->tickets;
    A.dev_error = h->dev_error;
#ifdef BORN_PROFILE
    if (const char* pp = getenv("BORN_PROF_PTR")) A.prof = (unsigned long long*)strtoull(pp, nullptr, 0);
#endif
    const int esz = a->logits_dtype == BORN_DTYPE_F32 ? 4 : 2;
    if (a->vocab_segments > 1) {
        A.S = a->vocab_segments;
        A.slice_len = a->vocab / a->vocab_segments;
        A.segment_mode = 1;
    } else {
        choose_slices(h, a->batch, a->vocab, esz, &A.S, &A.slice_len);
    }
    A.rec_row_stride = h->record_stride * A.S;
    A.tma_logits = ((uintptr_t)a->logits % 16 == 0) && ((a->logits_row_stride * esz) % 16 == 0) &&
                   (((int64_t)A.slice_len * esz) % 16 == 0);
    A.tma_mask = a->mask && ((uintptr_t)a->mask % 16 == 0) && ((a->mask_row_stride * 4) % 16 == 0) &&
                 (A.slice_len % 128 == 0);
    if (getenv("BORN_NO_TMA")) A.tma_logits = A.tma_mask = 0;
    return launch_sample(h, A, a->logits_dtype, st);
}

int32_t born_sample(void* handle, const born_sample_args* a, void* stream) {
    Handle* h = (Handle*)handle;
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    if (!a) return fail(h, BORN_ERR_INVALID_ARGUMENT, "args is NULL");
    if (a->struct_size != sizeof(born_sample_args))
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "struct_size %u != %zu", a->struct_size, sizeof(born_sample_args));
    if (a->batch <= 0 || a->vocab <= 0) return fail(h, BORN_ERR_INVALID_ARGUMENT, "batch and vocab must be positive");
    if (a->batch > h->max_batch || a->vocab > h->max_vocab)
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "batch %d / vocab %d exceed the handle's %d / %d", a->batch, a->vocab,
                    h->max_batch, h->max_vocab);
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
    if (a->out_kept_ids && a->kept_stride <= 0) return fail(h, BORN_ERR_INVALID_ARGUMENT, "kept_stride must be positive");
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
        if (a->mask && (a->vocab / G) % 32)
            return fail(h, BORN_ERR_UNSUPPORTED, "with a mask the segment length must be a multiple of 32");
        if ((int64_t)G * a->batch > h->max_records) return fail(h, BORN_ERR_UNSUPPORTED, "batch*segments exceeds the workspace");
    }
    CUDA_TRY(h, cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    if (a->memory == BORN_MEM_DEVICE) return sample_device(h, a, st);

    // ---- host-memory call: copy in, run, copy out, wait ----
    const int B = a->batch, V = a->vocab;
    const size_t esz = a->logits_dtype == BORN_DTYPE_F32 ? 4 : 2;
    const size_t words = (size_t)(V + 31) / 32;
    born_sample_args d = *a;
    d.memory = BORN_MEM_DEVICE;
    int rc;
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
    if ((rc = sample_device(h, &d, st))) return rc;
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
    CUDA_TRY(h, cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    SpecKernelArgs A;
    memset(&A, 0, sizeof A);
    A.B = B; A.K = K; A.V = V; A.target_rows = R;
    A.inv_T = a->temperature == 0.0f ? 1.0f : 1.0f / a->temperature;
    // scratch of the speculative path (tickets, chunk sums, block results): grown on first use
    // like the staging mirrors, then reused; the tickets are zero between launches
    const SpecScratchLayout SL = spec_scratch_layout(B, K, V);
    if (h->spec_scratch_bytes < SL.total) {
        CUDA_TRY(h, cudaStreamSynchronize(st));
        if (h->spec_scratch) { cudaFree(h->spec_scratch); h->workspace -= (int64_t)h->spec_scratch_bytes; h->spec_scratch = nullptr; h->spec_scratch_bytes = 0; }
        int rc0 = dev_alloc(h, (void**)&h->spec_scratch, SL.total);
        if (rc0 != BORN_OK) return rc0;
        h->spec_scratch_bytes = SL.total;
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
    CUDA_TRY(h, cudaSetDevice(h->device));
    Id128 u;
    memcpy(&u, id, sizeof u);
    int e = h->nccl.CommInitRank(&h->comm, nranks, u, rank);
    if (e != 0) return fail(h, BORN_ERR_NCCL, "ncclCommInitRank: %s", h->nccl.GetErrorString ? h->nccl.GetErrorString(e) : "error");
    h->rank = rank;
    h->nranks = nranks;
    return BORN_OK;
}

static int shard_check(Handle* h, const born_shard_args* a, bool local, bool merge) {
    if (!h) return fail(nullptr, BORN_ERR_INVALID_ARGUMENT, "handle is NULL");
    if (!a || a->struct_size != sizeof(born_shard_args)) return fail(h, BORN_ERR_INVALID_ARGUMENT, "args NULL or wrong struct_size");
    if (a->memory != BORN_MEM_DEVICE) return fail(h, BORN_ERR_UNSUPPORTED, "the sharded path takes device memory only");
    if (a->batch <= 0 || a->batch > h->max_batch || a->vocab_local <= 0 || a->vocab_local > h->max_vocab)
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "batch/vocab_local out of range");
    if (a->nranks < 1 || a->nranks > BORN_MAX_SHARDS || a->rank < 0 || a->rank >= a->nranks)
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "rank %d of %d", a->rank, a->nranks);
    if ((int64_t)a->vocab_local * a->nranks > BORN_MAX_VOCAB) return fail(h, BORN_ERR_UNSUPPORTED, "global vocab too large");
    if (a->top_k <= 0 || (int64_t)a->top_k * a->nranks > BORN_MAX_CANDIDATES)
        return fail(h, BORN_ERR_UNSUPPORTED, "need 1 <= top_k*nranks <= %d", BORN_MAX_CANDIDATES);
    if (!(a->temperature > 0.0f) || !isfinite(a->temperature) || !(a->top_p >= 0.0f))
        return fail(h, BORN_ERR_INVALID_ARGUMENT, "temperature must be > 0 and top_p >= 0");
    if (local) {
        if (!a->logits || a->logits_row_stride < a->vocab_local) return fail(h, BORN_ERR_INVALID_ARGUMENT, "logits");
        if (a->logits_dtype != BORN_DTYPE_F32 && a->logits_dtype != BORN_DTYPE_BF16) return fail(h, BORN_ERR_INVALID_ARGUMENT, "dtype");
    }
    if (merge && (!a->uniforms || !a->out_token || !a->out_status)) return fail(h, BORN_ERR_INVALID_ARGUMENT, "uniforms/out_token/out_status");
    return BORN_OK;
}

static void shard_fill(const born_shard_args* a, SampleKernelArgs& A, Handle* h) {
    memset(&A, 0, sizeof A);
    A.B = a->batch;
    A.params.temperature = a->temperature;
    A.params.top_p = a->top_p;
    A.params.top_k = a->top_k;
    A.params.repetition_penalty = 1.0f;
    A.uniforms = a->uniforms;
    A.out_token = a->out_token;
    A.out_prob = a->out_prob;
    A.out_lse = a->out_lse;
    A.out_status = a->out_status;
    A.tickets = h->tickets;
    A.dev_error = h->dev_error;
    A.segment_mode = 1;
}

static int shard_local(Handle* h, const born_shard_args* a, void* packed, bool want_lse, cudaStream_t st) {
    SampleKernelArgs A;
    shard_fill(a, A, h);
    const int esz = a->logits_dtype == BORN_DTYPE_F32 ? 4 : 2;
    A.logits = a->logits;
    A.row_stride = a->logits_row_stride;
    A.V = a->vocab_local;
    A.mode = kModeLocal;
    A.S = 1;
    A.slice_len = (a->vocab_local + kTileBytes / esz - 1) / (kTileBytes / esz) * (kTileBytes / esz);
    A.idx_offset = a->rank * a->vocab_local;
    A.records = (uint8_t*)packed;
    A.rec_row_stride = born_shard_record_bytes(a->top_k);
    A.rec_slice_stride = 0;
    A.tma_logits = ((uintptr_t)a->logits % 16 == 0) && ((a->logits_row_stride * esz) % 16 == 0);
    static float dummy_lse_flag;  // only its non-NULL-ness matters in local mode
    A.out_lse = want_lse ? &dummy_lse_flag : nullptr;
    A.out_token = nullptr;
    A.out_status = nullptr;
    return launch_sample(h, A, a->logits_dtype, st);
}

static int shard_merge(Handle* h, const born_shard_args* a, const void* gathered, cudaStream_t st) {
    SampleKernelArgs A;
    shard_fill(a, A, h);
    A.V = a->vocab_local * a->nranks;
    A.mode = kModeMerge;
    A.S = a->nranks;
    A.records = (uint8_t*)gathered;
    A.rec_row_stride = born_shard_record_bytes(a->top_k);
    A.rec_slice_stride = A.rec_row_stride * a->batch;
    return launch_sample(h, A, BORN_DTYPE_F32, st);
}

int32_t born_shard_local(void* handle, const born_shard_args* a, void* stream) {
    Handle* h = (Handle*)handle;
    int rc = shard_check(h, a, true, false);
    if (rc) return rc;
    if (!a->packed) return fail(h, BORN_ERR_INVALID_ARGUMENT, "packed is NULL");
    CUDA_TRY(h, cudaSetDevice(h->device));
    return shard_local(h, a, a->packed, true, (cudaStream_t)stream);
}

int32_t born_shard_merge(void* handle, const born_shard_args* a, void* stream) {
    Handle* h = (Handle*)handle;
    int rc = shard_check(h, a, false, true);
    if (rc) return rc;
    if (!a->gathered) return fail(h, BORN_ERR_INVALID_ARGUMENT, "gathered is NULL");
    CUDA_TRY(h, cudaSetDevice(h->device));
    return shard_merge(h, a, a->gathered, (cudaStream_t)stream);
}

int32_t born_sample_sharded(void* handle, const born_shard_args* a, void* stream) {
    Handle* h = (Handle*)handle;
    int rc = shard_check(h, a, true, true);
    if (rc) return rc;
    if (!h->comm) return fail(h, BORN_ERR_NCCL, "born_shard_init has not been called on this handle");
    if (a->nranks != h->nranks || a->rank != h->rank) return fail(h, BORN_ERR_INVALID_ARGUMENT, "rank/nranks differ from born_shard_init");
    CUDA_TRY(h, cudaSetDevice(h->device));
    cudaStream_t st = (cudaStream_t)stream;
    const size_t rec = (size_t)born_shard_record_bytes(a->top_k);
    const size_t pk = rec * (size_t)a->batch, ga = pk * (size_t)a->nranks;
    if (h->packed_bytes < pk) {  // grows once to the largest request seen
        cudaFree(h->packed); h->packed = nullptr; h->packed_bytes = 0;
        if ((rc = dev_alloc(h, (void**)&h->packed, pk))) return rc;
        h->packed_bytes = pk;
    }
    if (h->gathered_bytes < ga) {
        cudaFree(h->gathered); h->gathered = nullptr; h->gathered_bytes = 0;
        if ((rc = dev_alloc(h, (void**)&h->gathered, ga))) return rc;
        h->gathered_bytes = ga;
    }
    if ((rc = shard_local(h, a, h->packed, a->out_lse != nullptr, st))) return rc;
    int e = h->nccl.AllGather(h->packed, h->gathered, pk, /*ncclInt8*/ 0, h->comm, st);
    if (e != 0) return fail(h, BORN_ERR_NCCL, "ncclAllGather: %s", h->nccl.GetErrorString ? h->nccl.GetErrorString(e) : "error");
    return shard_merge(h, a, h->gathered, st);
}

}  // extern "C"

// ------------------------------------------------------------------ allocation-free entry
// Scratch for born_sample_static: slice records, row tickets and the device error word in
// one file-scope array that every GPU loading this library holds until exit.
namespace {
constexpr int kStaticMaxBatch = BORN_STATIC_MAX_BATCH;
constexpr int kStaticMaxRecords = 2 * BORN_STATIC_MAX_BATCH;
constexpr size_t kStaticRecordStride = kRecordHdrBytes + (size_t)kMaxK * 8;
constexpr size_t kStaticRecordsBytes = kStaticMaxRecords * kStaticRecordStride;
constexpr size_t kStaticTicketsBytes = sizeof(uint32_t) * 2 * kStaticMaxBatch;
constexpr size_t kStaticBytes = kStaticRecordsBytes + kStaticTicketsBytes + 256;
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
    if (a->vocab_segments > 1 && (int64_t)a->vocab_segments * a->batch > kStaticMaxRecords)
        return fail(nullptr, BORN_ERR_UNSUPPORTED, "born_sample_static: batch*vocab_segments exceeds %d scratch records",
                    kStaticMaxRecords);
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
        h->device = dev;
        h->is_static = true;
        h->max_batch = kStaticMaxBatch;
        h->max_vocab = BORN_MAX_VOCAB;
        h->max_k = BORN_MAX_TOP_K;
        h->num_sms = sms;
        h->max_records = kStaticMaxRecords;
        h->record_stride = (int64_t)kStaticRecordStride;
        h->records = base;
        h->tickets = reinterpret_cast<uint32_t*>(base + kStaticRecordsBytes);
        h->dev_error = reinterpret_cast<int*>(base + kStaticRecordsBytes + kStaticTicketsBytes);
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
