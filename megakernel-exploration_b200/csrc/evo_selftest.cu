// Unit check of the UMMA operand conventions (descriptor builders in
// evo_tiles.cuh) that the attention kernels rely on: one CTA multiplies small
// tiles through exactly the descriptors the real kernels use, and the host
// compares against a CPU GEMM.
#include "evo_host.cuh"
#include "evo_tiles.cuh"

namespace evo {

template <int DH>
__global__ void __launch_bounds__(128, 1)
selftest_mma_kernel(const __grid_constant__ CUtensorMap tm_y, const __grid_constant__ CUtensorMap tm_z,
                    const __nv_bfloat16* __restrict__ x, float* __restrict__ out_yzt,
                    float* __restrict__ out_xy, float* __restrict__ out_xty, float* __restrict__ out_ts,
                    unsigned int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sX = smem;                                // 32 KB square tile
    uint8_t* sY = sX + SQ_BYTES;                       // row tile
    uint8_t* sZ = sY + RowTile<DH>::BYTES;             // row tile
    uint64_t* bars = reinterpret_cast<uint64_t*>(sZ + RowTile<DH>::BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const int tid = threadIdx.x, warp = tid >> 5;
    WaitCtx wc{abort_flag, status};

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_init(&bars[2], 1);
        fence_mbar_init();
        fence_async_smem();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    // X: row `tid`, sixteen 16-byte chunks, into the swizzled square tile.
    {
        const uint4* src = reinterpret_cast<const uint4*>(x + tid * 128);
#pragma unroll
        for (int cc = 0; cc < 16; ++cc) {
            *reinterpret_cast<uint4*>(sX + sq_chunk_off(tid, cc)) = src[cc];
        }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    constexpr uint32_t T_A = 128 + 2 * DH;      // X as a bf16 A operand in tensor memory: 64 columns
    constexpr uint32_t T_TS = 0;                // its product with y: second phase, over the first product
    {
        // row `tid` of X: 64 words of two bf16 each, into this thread's lane
        const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16) + T_A;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(x + tid * 128);
        uint32_t r[32];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = src[h * 32 + i];
            tmem_st32(lane_addr + h * 32, r);
        }
        tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (tid == 0) {
        mbar_arrive_expect_tx(&bars[0], 2 * RowTile<DH>::BYTES);
        tma_load_row_tile<DH>(sY, &tm_y, &bars[0], 0, 0, 0);
        tma_load_row_tile<DH>(sZ, &tm_z, &bars[0], 0, 0, 0);
        if (mbar_wait(&bars[0], 0, wc, 1)) {
            tc_fence_after();
            const uint32_t aX = smem_u32(sX), aY = smem_u32(sY), aZ = smem_u32(sZ);
#pragma unroll
            for (int kb = 0; kb < RowTile<DH>::KBLOCKS; ++kb)
                umma_ss(tmem + 0, RowTile<DH>::kmajor(aY, kb), RowTile<DH>::kmajor(aZ, kb),
                        make_idesc_bf16(128, 128, 0, 0), kb > 0);
#pragma unroll
            for (int kb = 0; kb < 8; ++kb)
                umma_ss(tmem + 128, sq_kmajor(aX, kb), RowTile<DH>::mnmajor(aY, kb),
                        make_idesc_bf16(128, DH, 0, 1), kb > 0);
#pragma unroll
            for (int kb = 0; kb < 8; ++kb)
                umma_ss(tmem + 128 + DH, sq_mnmajor(aX, kb), RowTile<DH>::mnmajor(aY, kb),
                        make_idesc_bf16(128, DH, 1, 1), kb > 0);
            umma_commit(&bars[1]);
        }
    }
    __syncwarp();
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    if (warp_all(mbar_wait(&bars[1], 0, wc, 2))) {
        tc_fence_after();
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            tmem_ld32(lane_base + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) out_yzt[tid * 128 + c * 32 + i] = __uint_as_float(r[i]);
        }
#pragma unroll
        for (int c = 0; c < DH / 32; ++c) {
            tmem_ld32(lane_base + 128 + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) out_xy[tid * DH + c * 32 + i] = __uint_as_float(r[i]);
            tmem_ld32(lane_base + 128 + DH + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) out_xty[tid * DH + c * 32 + i] = __uint_as_float(r[i]);
        }
    }
    // second phase: the A operand from tensor memory, its product over the columns read above
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0 && *abort_flag == 0u) {
        const uint32_t aY = smem_u32(sY);
#pragma unroll
        for (int kb = 0; kb < 8; ++kb)
            umma_ts(tmem + T_TS, tmem + T_A + kb * 8, RowTile<DH>::mnmajor(aY, kb),
                    make_idesc_bf16(128, DH, 0, 1), kb > 0);
        umma_commit(&bars[2]);
    }
    __syncwarp();
    if (*abort_flag == 0u && warp_all(mbar_wait(&bars[2], 0, wc, 5))) {
        tc_fence_after();
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < DH / 32; ++c) {
            tmem_ld32(lane_base + T_TS + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) out_ts[tid * DH + c * 32 + i] = __uint_as_float(r[i]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

template <int DH>
static int launch_selftest(const void* x, const void* y, const void* z, float* o0, float* o1,
                           float* o2, float* o3, cudaStream_t st) {
    CUtensorMap tm_y, tm_z;
    int rc = make_tmap_qkv(&tm_y, y, 1, 128, 1, DH, 128, contiguous_layout(128, 1, DH), RowTile<DH>::BOX_D);
    if (rc) return rc;
    rc = make_tmap_qkv(&tm_z, z, 1, 128, 1, DH, 128, contiguous_layout(128, 1, DH), RowTile<DH>::BOX_D);
    if (rc) return rc;
    unsigned int* status = status_word();
    if (!status) return EVO_ERR_CUDA;
    const int smem = SQ_BYTES + 2 * RowTile<DH>::BYTES + 64 + 1024;
    rc = cuda_err(cudaFuncSetAttribute(selftest_mma_kernel<DH>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    if (rc) return rc;
    selftest_mma_kernel<DH><<<1, 128, smem, st>>>(tm_y, tm_z, static_cast<const __nv_bfloat16*>(x),
                                                   o0, o1, o2, o3, status);
    return cuda_err(cudaGetLastError());
}

// Extra contraction block (xt_desc, evo_tiles.cuh): out[128][128] = y z^T + a b^T with a, b
// [128][8] bf16 in the un-swizzled 16-byte-row layout and the second half of the block read
// from a zero tile.
template <int DH>
__global__ void __launch_bounds__(128, 1)
selftest_xt_kernel(const __grid_constant__ CUtensorMap tm_y, const __grid_constant__ CUtensorMap tm_z,
                   const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                   float* __restrict__ out, unsigned int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sY = smem;
    uint8_t* sZ = sY + RowTile<DH>::BYTES;
    uint8_t* sA = sZ + RowTile<DH>::BYTES;
    uint8_t* sB = sA + XT_BYTES;
    uint8_t* sZero = sB + XT_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sZero + XT_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const int tid = threadIdx.x, warp = tid >> 5;
    WaitCtx wc{abort_flag, status};
    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, 128);
        tmem_relinquish();
    }
    reinterpret_cast<uint4*>(sZero)[tid] = make_uint4(0u, 0u, 0u, 0u);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (tid == 0) {
        mbar_arrive_expect_tx(&bars[0], 2 * RowTile<DH>::BYTES + 2 * XT_BYTES);
        tma_load_row_tile<DH>(sY, &tm_y, &bars[0], 0, 0, 0);
        tma_load_row_tile<DH>(sZ, &tm_z, &bars[0], 0, 0, 0);
        bulk_load(sA, a, XT_BYTES, &bars[0]);
        bulk_load(sB, b, XT_BYTES, &bars[0]);
        if (mbar_wait(&bars[0], 0, wc, 3)) {
            tc_fence_after();
            const uint32_t aY = smem_u32(sY), aZ = smem_u32(sZ), aZero = smem_u32(sZero);
#pragma unroll
            for (int kb = 0; kb < RowTile<DH>::KBLOCKS; ++kb)
                umma_ss(tmem, RowTile<DH>::kmajor(aY, kb), RowTile<DH>::kmajor(aZ, kb),
                        make_idesc_bf16(128, 128, 0, 0), kb > 0);
            umma_ss(tmem, xt_desc(smem_u32(sA), aZero), xt_desc(smem_u32(sB), aZero),
                    make_idesc_bf16(128, 128, 0, 0), 1u);
            umma_commit(&bars[1]);
        }
    }
    __syncwarp();
    if (warp_all(mbar_wait(&bars[1], 0, wc, 4))) {
        tc_fence_after();
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            tmem_ld32(lane_base + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) out[tid * 128 + c * 32 + i] = __uint_as_float(r[i]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 128);
}

template <int DH>
static int launch_selftest_xt(const void* y, const void* z, const void* a, const void* b, float* out,
                              cudaStream_t st) {
    CUtensorMap tm_y, tm_z;
    int rc = make_tmap_qkv(&tm_y, y, 1, 128, 1, DH, 128, contiguous_layout(128, 1, DH), RowTile<DH>::BOX_D);
    if (rc) return rc;
    rc = make_tmap_qkv(&tm_z, z, 1, 128, 1, DH, 128, contiguous_layout(128, 1, DH), RowTile<DH>::BOX_D);
    if (rc) return rc;
    unsigned int* status = status_word();
    if (!status) return EVO_ERR_CUDA;
    const int smem = 2 * RowTile<DH>::BYTES + 3 * XT_BYTES + 64 + 1024;
    rc = cuda_err(cudaFuncSetAttribute(selftest_xt_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    if (rc) return rc;
    selftest_xt_kernel<DH><<<1, 128, smem, st>>>(tm_y, tm_z, static_cast<const __nv_bfloat16*>(a),
                                                  static_cast<const __nv_bfloat16*>(b), out, status);
    return cuda_err(cudaGetLastError());
}

// A wait that nothing will ever satisfy, with a short limit: warp 0 waits on an mbarrier
// nobody arrives at, gives up after `limit_ns`, records (ST_WAIT_TIMEOUT, site 0xee) in
// the status word and raises the CTA's abort flag; warp 1 waits on a second such barrier
// with the library's normal limits and must be released by the abort flag long before
// those run out.  Then the kernel returns normally: no trap, no fault, no unbounded spin.
__global__ void __launch_bounds__(64, 1) selftest_wait_kernel(unsigned long long limit_ns, unsigned int* status,
                                                              unsigned int* released) {
    __shared__ uint64_t bars[2];
    __shared__ uint32_t abort_word;
    volatile uint32_t* abort_flag = &abort_word;
    const int tid = threadIdx.x, warp = tid >> 5;
    WaitCtx wc{abort_flag, status};
    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        fence_mbar_init();
    }
    __syncthreads();
    bool ok;
    if (warp == 0) {
        ok = warp_all(mbar_wait_limited(&bars[0], 0, wc, 0xee, EVO_WAIT_LIMIT, limit_ns));
    } else {
        ok = warp_all(mbar_wait(&bars[1], 0, wc, 0xef));
        // released by the abort flag, not by its own limit: it never reports
        if (!ok && tid == 32) *released = (*abort_flag != 0u) ? 1u : 0u;
    }
    __syncthreads();
}

}  // namespace evo

extern "C" int evo_selftest_wait_timeout(unsigned long long limit_ns, unsigned int* released, void* stream) {
    if (!released) return EVO_ERR_NULL_PTR;
    if (limit_ns == 0 || limit_ns > 100000000ull) return EVO_ERR_BAD_DIMS;     // at most 0.1 s
    if (int rc = evo::ensure_context()) return rc;
    unsigned int* status = evo::status_word();
    if (!status) return EVO_ERR_CUDA;
    evo::selftest_wait_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns, status, released);
    return evo::cuda_err(cudaGetLastError());
}

extern "C" int evo_selftest_mma_extra(int D, const void* y, const void* z, const void* a, const void* b,
                                      float* out, void* stream) {
    if (!y || !z || !a || !b || !out) return EVO_ERR_NULL_PTR;
    if (D != 32 && D != 64 && D != 128) return EVO_ERR_BAD_DIMS;
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15u) return EVO_ERR_ALIGNMENT;
    if (int rc = evo::ensure_context()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (D == 32) return evo::launch_selftest_xt<32>(y, z, a, b, out, st);
    if (D == 64) return evo::launch_selftest_xt<64>(y, z, a, b, out, st);
    return evo::launch_selftest_xt<128>(y, z, a, b, out, st);
}

extern "C" int evo_selftest_mma(int D, const void* x, const void* y, const void* z, float* out_yzt,
                                float* out_xy, float* out_xty, float* out_ts, void* stream) {
    if (!x || !y || !z || !out_yzt || !out_xy || !out_xty || !out_ts) return EVO_ERR_NULL_PTR;
    if (D != 32 && D != 64 && D != 128) return EVO_ERR_BAD_DIMS;
    if (int rc = evo::ensure_context()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (D == 32) return evo::launch_selftest<32>(x, y, z, out_yzt, out_xy, out_xty, out_ts, st);
    if (D == 64) return evo::launch_selftest<64>(x, y, z, out_yzt, out_xy, out_xty, out_ts, st);
    if (D == 128) return evo::launch_selftest<128>(x, y, z, out_yzt, out_xy, out_xty, out_ts, st);
    return EVO_ERR_BAD_DIMS;
}
