// Host-side helpers shared by the launchers: error codes, the driver entry
// point for tensor-map encoding (resolved at run time so the library has no
// link-time dependency on libcuda), and tensor-map builders for the layouts
// this library reads and writes.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/evoattn.h"

namespace evo {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Returns nullptr when no CUDA driver is present.
EncodeTiledFn encode_tiled_fn();

struct TmapDim {
    uint64_t extent;       // elements
    uint64_t stride_bytes; // ignored for dim 0 (contiguous)
    uint32_t box;          // elements
};

// rank <= 5; dims[0] is the contiguous one.  Returns EVO_OK or an error code.
int make_tmap(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int rank,
              const TmapDim* dims, CUtensorMapSwizzle swz);

inline CUtensorMapSwizzle row_swizzle(int D) {
    return D == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
}

// Element strides of an activation tensor over (flattened B*S row, residue, head); D is contiguous.
struct ActLayout {
    long long row, n, h;
};
inline ActLayout contiguous_layout(int N, int H, int D) {
    return ActLayout{static_cast<long long>(N) * H * D, static_cast<long long>(H) * D, static_cast<long long>(D)};
}
// Checks EvoStrides against the rules of the header and flattens (B, S); NULL = contiguous.
int layout_from_strides(const EvoDims* d, const EvoStrides* s, ActLayout* out);

// bf16 activation tensor viewed as (D, H, N, BS) with the strides of `lay`; box = one
// head's [rows x box_d] tile (box_d = 0: D), swizzled by box row.  A box wider than D (D = 16
// read by the D = 32 kernels) is zero-filled past D on loads and clipped on stores.
int make_tmap_qkv(CUtensorMap* out, const void* base, int BS, int N, int H, int D, int rows,
                  const ActLayout& lay, int box_d = 0);
// The same view with a box of [rows x cols] head-dim columns (cols * 2 bytes = 32, 64 or 128), swizzled by box row.
int make_tmap_qkv_cols(CUtensorMap* out, const void* base, int BS, int N, int H, int D, int rows, int cols,
                       const ActLayout& lay);
// [BS][N][H][D] of `elem_bytes`-wide elements (2: bf16, 4: fp32) with a box of
// [rows x box_cols]; the swizzle matches the box row (32, 64 or 128 bytes).
int make_tmap_rows_box(CUtensorMap* out, const void* base, int elem_bytes, int BS, int N, int H, int D,
                       int box_cols, int rows);
// fp32 [B][H][N][N] with a box of [rows x box_cols], swizzle by box row bytes.
int make_tmap_dbias_box(CUtensorMap* out, const void* base, int B, int H, int N, int box_cols, int rows);
// bf16 [B][H][N][N] viewed as (N, N, H, B); box [128 rows x 64 cols], 128B swizzle.
int make_tmap_bias(CUtensorMap* out, const void* base, int B, int H, int N);

int check_dims(const EvoDims* d);
// Makes the device's primary context current on this thread (see evo_host.cu).
int ensure_context();
// Device address of this device's status word (nullptr on failure).
unsigned int* status_word();
int cuda_err(cudaError_t e);
// SM count of the current device (read once per device).
int sm_count(int* out);
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (device, kernel, size).
int set_max_smem_once(const void* func, int bytes);

// Event pairs around the main kernels when profiling is enabled (no-ops otherwise).
void prof_begin(int kernel, cudaStream_t st);
void prof_end(int kernel, cudaStream_t st);

}  // namespace evo
