// Host-side helpers: error strings, argument checks, tensor-map construction,
// the device status word.
#include "evo_host.cuh"

#include <cstdio>
#include <mutex>
#include <vector>

namespace evo {

static thread_local int t_last_cuda_error = 0;
static thread_local char t_detail[512] = "";

int cuda_err(cudaError_t e) {
    if (e == cudaSuccess) return EVO_OK;
    t_last_cuda_error = static_cast<int>(e);
    (void)cudaGetLastError();  // clear the sticky-less error state
    return EVO_ERR_CUDA;
}

EncodeTiledFn encode_tiled_fn() {
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        } else {
            (void)cudaGetLastError();
        }
    });
    return fn;
}

namespace {
// Encoded tensor maps keyed on everything the encoder sees.  A training loop calls with the same few
// (pointer, shape, strides) combinations step after step; encoding costs microseconds per map on the
// host, a dozen maps per step.  The cache is small and evicts round-robin.
struct TmapKey {
    const void* base;
    int dt, rank, swz;
    uint64_t extent[5], stride[5];
    uint32_t box[5];
    bool operator==(const TmapKey& o) const {
        if (base != o.base || dt != o.dt || rank != o.rank || swz != o.swz) return false;
        for (int i = 0; i < rank; ++i)
            if (extent[i] != o.extent[i] || stride[i] != o.stride[i] || box[i] != o.box[i]) return false;
        return true;
    }
};
struct TmapEntry {
    TmapKey key;
    CUtensorMap map;
};
constexpr size_t TMAP_CACHE = 256;
std::mutex g_tmap_mu;
std::vector<TmapEntry> g_tmap_cache;
size_t g_tmap_next = 0;
}  // namespace

static int encode_tmap(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int rank,
                       const TmapDim* dims, CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return EVO_ERR_NO_DRIVER;
    cuuint64_t extent[5];
    cuuint64_t stride[5];
    cuuint32_t box[5];
    cuuint32_t estr[5];
    for (int i = 0; i < rank; ++i) {
        extent[i] = dims[i].extent;
        box[i] = dims[i].box;
        estr[i] = 1;
        if (i > 0) stride[i - 1] = dims[i].stride_bytes;
    }
    CUresult r = fn(out, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), extent, stride,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) return EVO_OK;
    int n = snprintf(t_detail, sizeof(t_detail), "cuTensorMapEncodeTiled -> %d: base=%p dtype=%d rank=%d swizzle=%d",
                     static_cast<int>(r), base, static_cast<int>(dt), rank, static_cast<int>(swz));
    for (int i = 0; i < rank && n > 0 && n < static_cast<int>(sizeof(t_detail)); ++i)
        n += snprintf(t_detail + n, sizeof(t_detail) - n, " [extent=%llu stride=%llu box=%u]",
                      static_cast<unsigned long long>(dims[i].extent),
                      static_cast<unsigned long long>(i > 0 ? dims[i].stride_bytes : 0), dims[i].box);
    return EVO_ERR_TENSOR_MAP;
}

int make_tmap(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int rank,
              const TmapDim* dims, CUtensorMapSwizzle swz) {
    if (rank < 1 || rank > 5) return EVO_ERR_TENSOR_MAP;
    TmapKey key{};
    key.base = base; key.dt = static_cast<int>(dt); key.rank = rank; key.swz = static_cast<int>(swz);
    for (int i = 0; i < rank; ++i) {
        key.extent[i] = dims[i].extent;
        key.stride[i] = i > 0 ? dims[i].stride_bytes : 0;
        key.box[i] = dims[i].box;
    }
    {
        std::lock_guard<std::mutex> lock(g_tmap_mu);
        for (const TmapEntry& e : g_tmap_cache)
            if (e.key == key) { *out = e.map; return EVO_OK; }
    }
    // A tensor map holds a virtual address and a shape, nothing device-specific: an entry encoded
    // while one device was current is valid for the same pointer under any other.
    const int rc = encode_tmap(out, base, dt, rank, dims, swz);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(g_tmap_mu);
    if (g_tmap_cache.size() < TMAP_CACHE) {
        g_tmap_cache.push_back(TmapEntry{key, *out});
    } else {
        g_tmap_cache[g_tmap_next] = TmapEntry{key, *out};
        g_tmap_next = (g_tmap_next + 1) % TMAP_CACHE;
    }
    return EVO_OK;
}

int make_tmap_qkv(CUtensorMap* out, const void* base, int BS, int N, int H, int D, int rows,
                  const ActLayout& lay, int box_d) {
    const uint64_t e = 2;
    if (box_d <= 0) box_d = D;
    TmapDim d[4] = {
        {static_cast<uint64_t>(D), 0, static_cast<uint32_t>(box_d)},
        {static_cast<uint64_t>(H), static_cast<uint64_t>(lay.h) * e, 1},
        {static_cast<uint64_t>(N), static_cast<uint64_t>(lay.n) * e, static_cast<uint32_t>(rows)},
        {static_cast<uint64_t>(BS), static_cast<uint64_t>(lay.row) * e, 1},
    };
    return make_tmap(out, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, d, row_swizzle(box_d));
}

int make_tmap_qkv_cols(CUtensorMap* out, const void* base, int BS, int N, int H, int D, int rows, int cols,
                       const ActLayout& lay) {
    const uint64_t e = 2;
    const int rb = cols * 2;
    if (rb != 16 && rb != 32 && rb != 64 && rb != 128) return EVO_ERR_TENSOR_MAP;
    TmapDim d[4] = {
        {static_cast<uint64_t>(D), 0, static_cast<uint32_t>(cols)},
        {static_cast<uint64_t>(H), static_cast<uint64_t>(lay.h) * e, 1},
        {static_cast<uint64_t>(N), static_cast<uint64_t>(lay.n) * e, static_cast<uint32_t>(rows)},
        {static_cast<uint64_t>(BS), static_cast<uint64_t>(lay.row) * e, 1},
    };
    const CUtensorMapSwizzle sw = rb == 16 ? CU_TENSOR_MAP_SWIZZLE_NONE
                                : (rb == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                : (rb == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B));
    return make_tmap(out, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, d, sw);
}

int layout_from_strides(const EvoDims* d, const EvoStrides* s, ActLayout* out) {
    if (!s) {
        *out = contiguous_layout(d->N, d->H, d->D);
        return EVO_OK;
    }
    const long long st[4] = {s->b, s->s, s->n, s->h};
    const int ext[4] = {d->B, d->S, d->N, d->H};
    for (int i = 0; i < 4; ++i)      // an axis of extent 1 may carry any stride
        if (ext[i] > 1 && (st[i] <= 0 || st[i] % 8 != 0)) return EVO_ERR_BAD_DIMS;
    if (d->B > 1 && d->S > 1 && s->b != static_cast<long long>(d->S) * s->s) return EVO_ERR_BAD_DIMS;
    out->row = (d->S > 1) ? s->s : ((d->B > 1) ? s->b : static_cast<long long>(d->N) * d->H * d->D);
    out->n = (d->N > 1) ? s->n : static_cast<long long>(d->H) * d->D;
    out->h = (d->H > 1) ? s->h : static_cast<long long>(d->D);
    if (out->row % 8 || out->n % 8 || out->h % 8) return EVO_ERR_BAD_DIMS;
    return EVO_OK;
}

int make_tmap_bias(CUtensorMap* out, const void* base, int B, int H, int N) {
    const uint64_t e = 2;
    TmapDim d[4] = {
        {static_cast<uint64_t>(N), 0, 64},
        {static_cast<uint64_t>(N), N * e, 128},
        {static_cast<uint64_t>(H), static_cast<uint64_t>(N) * N * e, 1},
        {static_cast<uint64_t>(B), static_cast<uint64_t>(H) * N * N * e, 1},
    };
    return make_tmap(out, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, d, CU_TENSOR_MAP_SWIZZLE_128B);
}

static CUtensorMapSwizzle swizzle_for(int row_bytes) {
    return row_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                           : (row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
}

int make_tmap_rows_box(CUtensorMap* out, const void* base, int elem_bytes, int BS, int N, int H, int D,
                       int box_cols, int rows) {
    const uint64_t e = static_cast<uint64_t>(elem_bytes);
    const int rb = box_cols * elem_bytes;
    if (rb != 32 && rb != 64 && rb != 128) return EVO_ERR_TENSOR_MAP;
    TmapDim d[4] = {
        {static_cast<uint64_t>(D), 0, static_cast<uint32_t>(box_cols)},
        {static_cast<uint64_t>(H), D * e, 1},
        {static_cast<uint64_t>(N), static_cast<uint64_t>(H) * D * e, static_cast<uint32_t>(rows)},
        {static_cast<uint64_t>(BS), static_cast<uint64_t>(N) * H * D * e, 1},
    };
    return make_tmap(out, base, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                     4, d, swizzle_for(rb));
}

int make_tmap_dbias_box(CUtensorMap* out, const void* base, int B, int H, int N, int box_cols, int rows) {
    const uint64_t e = 4;
    const int rb = box_cols * 4;
    if (rb != 32 && rb != 64 && rb != 128) return EVO_ERR_TENSOR_MAP;
    TmapDim d[4] = {
        {static_cast<uint64_t>(N), 0, static_cast<uint32_t>(box_cols)},
        {static_cast<uint64_t>(N), N * e, static_cast<uint32_t>(rows)},
        {static_cast<uint64_t>(H), static_cast<uint64_t>(N) * N * e, 1},
        {static_cast<uint64_t>(B), static_cast<uint64_t>(H) * N * N * e, 1},
    };
    return make_tmap(out, base, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, d, swizzle_for(rb));
}

// Binds the device's primary context to the calling thread.  The tensor-map
// encoder is a driver call and fails with "invalid context" on a thread (for
// example an autograd worker) that has not made a runtime call yet.
int ensure_context() {
    int dev = 0;
    int rc = cuda_err(cudaGetDevice(&dev));
    if (rc) return rc;
    return cuda_err(cudaSetDevice(dev));
}

// One status word per device; kernels receive its address as an argument.
#ifdef EVO_TRACE
__device__ unsigned long long g_status_word[1 + 512 + 8 * 64 * 8] = {0};   // status word + cycle accounting + timeline
#else
__device__ unsigned int g_status_word = 0;
#endif

unsigned int* status_word() {
    static std::mutex mu;
    static unsigned int* cache[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        (void)cudaGetLastError();
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!cache[dev]) {
        void* p = nullptr;
        if (cuda_err(cudaGetSymbolAddress(&p, g_status_word)) != EVO_OK) return nullptr;
        cache[dev] = static_cast<unsigned int*>(p);
    }
    return cache[dev];
}

// ---- optional per-kernel timing ------------------------------------------------
namespace {
struct ProfRec {
    std::vector<cudaEvent_t> start, stop;
    bool armed = false;      // prof_begin pushed a pair that prof_end has not closed yet
};
std::mutex g_prof_mu;
bool g_prof_on = false;
ProfRec g_prof[3];
constexpr size_t PROF_MAX = 4096;
}  // namespace

void prof_begin(int kernel, cudaStream_t st) {
    std::lock_guard<std::mutex> lock(g_prof_mu);
    ProfRec& r = g_prof[kernel];
    r.armed = false;
    if (!g_prof_on || r.start.size() >= PROF_MAX) return;
    cudaEvent_t a = nullptr, b = nullptr;
    if (cudaEventCreate(&a) != cudaSuccess) {
        (void)cudaGetLastError();
        return;
    }
    if (cudaEventCreate(&b) != cudaSuccess) {
        (void)cudaGetLastError();
        cudaEventDestroy(a);
        return;
    }
    cudaEventRecord(a, st);
    r.start.push_back(a);
    r.stop.push_back(b);
    r.armed = true;
}

void prof_end(int kernel, cudaStream_t st) {
    std::lock_guard<std::mutex> lock(g_prof_mu);
    ProfRec& r = g_prof[kernel];
    if (!r.armed) return;        // the matching prof_begin recorded nothing (off, full, or failed)
    cudaEventRecord(r.stop.back(), st);
    r.armed = false;
}

// ---- per-device launch constants and the tensor-map cache ---------------------------
int sm_count(int* out) {
    static std::mutex mu;
    static int cache[64] = {0};
    int dev = 0;
    int rc = cuda_err(cudaGetDevice(&dev));
    if (rc) return rc;
    if (dev < 0 || dev >= 64) return EVO_ERR_CUDA;
    std::lock_guard<std::mutex> lock(mu);
    if (!cache[dev]) {
        int sms = 0;
        if ((rc = cuda_err(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)))) return rc;
        cache[dev] = sms;
    }
    *out = cache[dev];
    return EVO_OK;
}

int set_max_smem_once(const void* func, int bytes) {
    // one attribute call per (device, kernel): the key is the pair, the value the size last set
    struct Key { int dev; const void* fn; int bytes; };
    static std::mutex mu;
    static std::vector<Key> done;
    int dev = 0;
    int rc = cuda_err(cudaGetDevice(&dev));
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(mu);
    for (const Key& k : done)
        if (k.dev == dev && k.fn == func && k.bytes == bytes) return EVO_OK;
    if ((rc = cuda_err(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes)))) return rc;
    done.push_back(Key{dev, func, bytes});
    return EVO_OK;
}


int check_dims(const EvoDims* d) {
    if (!d) return EVO_ERR_NULL_PTR;
    if (d->B <= 0 || d->S <= 0 || d->N <= 0 || d->H <= 0) return EVO_ERR_BAD_DIMS;
    if (d->D != 16 && d->D != 32 && d->D != 64 && d->D != 96 && d->D != 128) return EVO_ERR_BAD_DIMS;
    if (d->N % 8 != 0) return EVO_ERR_BAD_DIMS;
    const double bytes = 2.0 * d->B * d->S * d->N * d->H * d->D;
    if (bytes >= 1099511627776.0) return EVO_ERR_BAD_DIMS;
    if (static_cast<double>(d->B) * d->S * d->H * ((d->N + 127) / 128) >= 2147483647.0)
        return EVO_ERR_BAD_DIMS;
    return EVO_OK;
}

}  // namespace evo

extern "C" {

int evo_version(void) { return 103; }

int evo_last_cuda_error(void) { return evo::t_last_cuda_error; }

const char* evo_last_error_detail(void) { return evo::t_detail; }

int evo_device_status(uint32_t* raw) {
    unsigned int* p = evo::status_word();
    if (!p) return EVO_ERR_CUDA;
    unsigned int v = 0;
    int rc = evo::cuda_err(cudaDeviceSynchronize());
    if (rc) return rc;
    rc = evo::cuda_err(cudaMemcpy(&v, p, sizeof(v), cudaMemcpyDeviceToHost));
    if (rc) return rc;
    if (raw) *raw = v;
    if (v == 0) return EVO_OK;
    rc = evo::cuda_err(cudaMemset(p, 0, sizeof(v)));
    if (rc) return rc;
    return EVO_ERR_DEVICE_WAIT;
}

#ifdef EVO_TRACE
// Trace builds only: copies (and clears) the 256 (cycles, count) pairs.
int evo_trace_read(unsigned long long* out) {
    unsigned int* p = evo::status_word();
    if (!p) return EVO_ERR_CUDA;
    int rc = evo::cuda_err(cudaDeviceSynchronize());
    if (rc) return rc;
    rc = evo::cuda_err(cudaMemcpy(out, p + 2, 512 * 8, cudaMemcpyDeviceToHost));
    if (rc) return rc;
    return evo::cuda_err(cudaMemset(p + 2, 0, 512 * 8));
}
// Trace builds only: copies (and clears) the timeline of CTA 0: [8 roles][64 steps][8 events] clock values.
int evo_timeline_read(unsigned long long* out) {
    unsigned int* p = evo::status_word();
    if (!p) return EVO_ERR_CUDA;
    int rc = evo::cuda_err(cudaDeviceSynchronize());
    if (rc) return rc;
    rc = evo::cuda_err(cudaMemcpy(out, p + 2 + 1024, 8 * 64 * 8 * 8, cudaMemcpyDeviceToHost));
    if (rc) return rc;
    return evo::cuda_err(cudaMemset(p + 2 + 1024, 0, 8 * 64 * 8 * 8));
}
#endif

int evo_profile_enable(int on) {
    std::lock_guard<std::mutex> lock(evo::g_prof_mu);
    evo::g_prof_on = (on != 0);
    return EVO_OK;
}

int evo_profile_read(int kernel, float* total_ms, int* launches) {
    if (kernel < 0 || kernel > 2 || !total_ms || !launches) return EVO_ERR_NULL_PTR;
    std::lock_guard<std::mutex> lock(evo::g_prof_mu);
    evo::ProfRec& r = evo::g_prof[kernel];
    float sum = 0.f;
    int n = 0, rc = EVO_OK;
    for (size_t i = 0; i < r.start.size(); ++i) {
        float ms = 0.f;
        if (cudaEventSynchronize(r.stop[i]) == cudaSuccess &&
            cudaEventElapsedTime(&ms, r.start[i], r.stop[i]) == cudaSuccess) {
            sum += ms;
            ++n;
        } else {
            (void)cudaGetLastError();
            rc = EVO_ERR_CUDA;
        }
        cudaEventDestroy(r.start[i]);
        cudaEventDestroy(r.stop[i]);
    }
    r.start.clear();
    r.stop.clear();
    *total_ms = sum;
    *launches = n;
    return rc;
}

const char* evo_strerror(int code) {
    switch (code) {
        case EVO_OK: return "ok";
        case EVO_ERR_BAD_DIMS: return "unsupported dimensions (need D in {16,32,64,96,128}, N % 8 == 0)";
        case EVO_ERR_NULL_PTR: return "null pointer argument";
        case EVO_ERR_ALIGNMENT: return "pointer not 16-byte aligned";
        case EVO_ERR_WORKSPACE: return "workspace too small or misaligned";
        case EVO_ERR_NO_DRIVER: return "CUDA driver entry point cuTensorMapEncodeTiled unavailable";
        case EVO_ERR_TENSOR_MAP: return "tensor-map encoding failed";
        case EVO_ERR_CUDA: return "CUDA runtime error";
        case EVO_ERR_DEVICE_WAIT: return "a kernel's bounded wait ran out";
        case EVO_ERR_TOO_LARGE: return "problem exceeds the capacity of this entry point";
        default: return "unknown error";
    }
}

}  // extern "C"
