// Host-side helpers: error strings, argument checks, tensor-map construction,
// the device status word.
#include "evo_host.cuh"

#include <mutex>

namespace evo {

static thread_local int t_last_cuda_error = 0;

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

int make_tmap(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int rank,
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
    return r == CUDA_SUCCESS ? EVO_OK : EVO_ERR_TENSOR_MAP;
}

int make_tmap_qkv(CUtensorMap* out, const void* base, int BS, int N, int H, int D, int rows) {
    const uint64_t e = 2;
    TmapDim d[4] = {
        {static_cast<uint64_t>(D), 0, static_cast<uint32_t>(D)},
        {static_cast<uint64_t>(H), D * e, 1},
        {static_cast<uint64_t>(N), static_cast<uint64_t>(H) * D * e, static_cast<uint32_t>(rows)},
        {static_cast<uint64_t>(BS), static_cast<uint64_t>(N) * H * D * e, 1},
    };
    return make_tmap(out, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, d, row_swizzle(D));
}

int make_tmap_qkv_f32(CUtensorMap* out, const void* base, int BS, int N, int H, int D, int rows) {
    const uint64_t e = 4;
    TmapDim d[4] = {
        {static_cast<uint64_t>(D), 0, 32},
        {static_cast<uint64_t>(H), D * e, 1},
        {static_cast<uint64_t>(N), static_cast<uint64_t>(H) * D * e, static_cast<uint32_t>(rows)},
        {static_cast<uint64_t>(BS), static_cast<uint64_t>(N) * H * D * e, 1},
    };
    return make_tmap(out, base, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, d, CU_TENSOR_MAP_SWIZZLE_128B);
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

int make_tmap_dbias(CUtensorMap* out, const void* base, int B, int H, int N) {
    const uint64_t e = 4;
    TmapDim d[4] = {
        {static_cast<uint64_t>(N), 0, 32},
        {static_cast<uint64_t>(N), N * e, 128},
        {static_cast<uint64_t>(H), static_cast<uint64_t>(N) * N * e, 1},
        {static_cast<uint64_t>(B), static_cast<uint64_t>(H) * N * N * e, 1},
    };
    return make_tmap(out, base, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, d, CU_TENSOR_MAP_SWIZZLE_128B);
}

// One status word per device; kernels receive its address as an argument.
__device__ unsigned int g_status_word = 0;

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

int check_dims(const EvoDims* d) {
    if (!d) return EVO_ERR_NULL_PTR;
    if (d->B <= 0 || d->S <= 0 || d->N <= 0 || d->H <= 0) return EVO_ERR_BAD_DIMS;
    if (d->D != 32 && d->D != 64) return EVO_ERR_BAD_DIMS;
    if (d->N % 8 != 0) return EVO_ERR_BAD_DIMS;
    const double bytes = 2.0 * d->B * d->S * d->N * d->H * d->D;
    if (bytes >= 1099511627776.0) return EVO_ERR_BAD_DIMS;
    if (static_cast<double>(d->B) * d->S * d->H * ((d->N + 127) / 128) >= 2147483647.0)
        return EVO_ERR_BAD_DIMS;
    return EVO_OK;
}

}  // namespace evo

extern "C" {

int evo_version(void) { return 100; }

int evo_last_cuda_error(void) { return evo::t_last_cuda_error; }

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

const char* evo_strerror(int code) {
    switch (code) {
        case EVO_OK: return "ok";
        case EVO_ERR_BAD_DIMS: return "unsupported dimensions (need D in {32,64}, N % 8 == 0)";
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
