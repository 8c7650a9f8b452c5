// Shared-memory tile conventions used by every kernel of this library, and the
// UMMA descriptors that address them.
//
// ROW TILE  [R rows][DH bf16], DH in {32, 64, 128}: what one TMA box load (DH = 128:
//   two box loads of 64 columns) of a q/k/v/dO tile produces.  DH <= 64: row pitch
//   2*DH bytes (64 B or 128 B), swizzled with the matching TMA mode (SWIZZLE_64B /
//   SWIZZLE_128B); the tile base is 1024-byte aligned.  DH = 128: two sub-tiles of
//   [128 rows][64 bf16], 16 KB apart, each laid out like the DH = 64 tile (the layout
//   of the square tile below).
//     * as a K-major operand  (rows index M or N, DH is the contraction axis)
//     * as an MN-major operand (rows index K, DH is the M or N axis; at DH = 128 the
//       two 64-wide swizzle atoms are reached through the leading-dimension offset)
//
// SQUARE TILE [128 rows][128 bf16]: P / dS, written by threads.  Stored as two
//   sub-tiles of [128 rows][64 bf16] (16 KB each, 128-byte rows, 128B swizzle):
//   16-byte chunk c of row r of sub-tile t sits at
//       t*16384 + r*128 + ((c ^ (r & 7)) << 4).
//     * as a K-major A operand  (rows = M, columns = K)
//     * as an MN-major A operand (rows = K, columns = M)
#pragma once
#include "evo_ptx.cuh"

namespace evo {

constexpr int TILE = 128;                 // q rows and kv rows per tile
constexpr uint32_t SQ_SUB_BYTES = 16384;  // one [128][64] bf16 sub-tile
constexpr uint32_t SQ_BYTES = 2 * SQ_SUB_BYTES;

template <int DH>
struct RowTile {
    static_assert(DH == 32 || DH == 64 || DH == 128, "head dim 32, 64 or 128");
    static constexpr int SUBS = (DH == 128) ? 2 : 1;     // sub-tiles of BOX_D columns
    static constexpr int BOX_D = DH / SUBS;              // columns of one TMA box
    static constexpr uint32_t ROW_BYTES = BOX_D * 2;     // row pitch inside a sub-tile
    static constexpr uint32_t SWZ = (DH == 32) ? SWZ_64B : SWZ_128B;
    static constexpr uint32_t SBO = 8 * ROW_BYTES;       // eight rows
    static constexpr uint32_t SUB_BYTES = TILE * ROW_BYTES;
    static constexpr uint32_t BYTES = SUBS * SUB_BYTES;  // 128-row tile
    static constexpr int KBLOCKS = DH / 16;              // UMMA K = 16 for bf16

    // K-major operand, contraction block kb (16 bf16 = 32 bytes along the row; four blocks per sub-tile).
    __device__ static __forceinline__ uint64_t kmajor(uint32_t saddr, int kb) {
        return make_smem_desc(saddr + (kb >> 2) * SUB_BYTES + (kb & 3) * 32, 16, SBO, SWZ);
    }
    // MN-major operand, contraction block kb = rows 16*kb .. 16*kb+15.
    __device__ static __forceinline__ uint64_t mnmajor(uint32_t saddr, int kb) {
        return make_smem_desc(saddr + kb * 16 * ROW_BYTES, SUB_BYTES, SBO, SWZ);
    }
};

// One row tile by TMA: box (BOX_D columns, one head, 128 rows, one row of B*S) per sub-tile.
template <int DH>
__device__ __forceinline__ void tma_load_row_tile(void* dst, const CUtensorMap* tm, uint64_t* bar, int h, int n0,
                                                  int bs) {
#pragma unroll
    for (int s = 0; s < RowTile<DH>::SUBS; ++s)
        tma_load_4d(static_cast<uint8_t*>(dst) + s * RowTile<DH>::SUB_BYTES, tm, bar, s * RowTile<DH>::BOX_D, h, n0, bs);
}

// Byte offset of the 16-byte chunk `cc` (0..15, eight bf16 columns each) of row r.
__device__ __forceinline__ uint32_t sq_chunk_off(int r, int cc) {
    return (cc >> 3) * SQ_SUB_BYTES + r * 128 + (((cc & 7) ^ (r & 7)) << 4);
}
// Square tile as K-major A: contraction block kb (0..7) = columns 16*kb..16*kb+15.
__device__ __forceinline__ uint64_t sq_kmajor(uint32_t saddr, int kb) {
    return make_smem_desc(saddr + (kb >> 2) * SQ_SUB_BYTES + (kb & 3) * 32, 16, 1024, SWZ_128B);
}
// Square tile as MN-major A (M = the 128 columns, two 64-wide swizzle atoms
// SQ_SUB_BYTES apart): contraction block kb (0..7) = rows 16*kb..16*kb+15.
__device__ __forceinline__ uint64_t sq_mnmajor(uint32_t saddr, int kb) {
    return make_smem_desc(saddr + kb * 16 * 128, SQ_SUB_BYTES, 1024, SWZ_128B);
}

// EXTRA TILE [128 rows][8 bf16]: 16-byte rows, dense (2 KB): the canonical un-swizzled
//   K-major layout with one 16-byte chunk per row (eight rows = one contiguous 128-byte
//   core matrix).  A UMMA contraction block is 16 bf16 = two chunks; the second chunk
//   (k = 8..15) is read from a zero-filled 2 KB tile at a HIGHER shared address, reached
//   through the descriptor's leading-dimension offset.  An extra tile appended to a
//   contraction adds rank-8 terms a[m, 0..7] . b[n, 0..7] to the product: per-row and
//   per-column additive terms (mask, -LSE, -delta) then come out of the tensor core
//   already summed into the logits instead of costing an add per element.
constexpr uint32_t XT_BYTES = 2048;
__device__ __forceinline__ uint64_t xt_desc(uint32_t saddr, uint32_t zero_saddr) {
    return make_smem_desc(saddr, zero_saddr - saddr, 128, SWZ_NONE);
}

// ---- split descriptors -------------------------------------------------------------
// The thread that issues MMAs is a single thread: every integer instruction it
// spends on building a descriptor delays the next MMA.  A descriptor's upper
// word is a compile-time constant per operand kind, and its lower word is
// (address >> 4) plus a constant, so an operand is addressed by ONE add on a
// lower word prepared once per tile:  desc = {hi, lo_base + (byte offset >> 4)}.
// (Shared-memory addresses are below 2^18, so address >> 4 fits the 14-bit field.)
__device__ __forceinline__ uint64_t desc_join(uint32_t lo, uint32_t hi) {
    return (static_cast<uint64_t>(hi) << 32) | lo;
}
__host__ __device__ constexpr uint32_t desc_hi(uint32_t sbo_bytes, uint32_t swz) {
    return ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | ((swz & 7u) << 29);
}
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
    return (saddr >> 4) | ((lbo_bytes >> 4) << 16);
}

template <int DH>
struct RowDesc {
    using RT = RowTile<DH>;
    static constexpr uint32_t HI = desc_hi(RT::SBO, RT::SWZ);
    __device__ static __forceinline__ uint32_t kmajor_lo(uint32_t saddr) { return desc_lo(saddr, 16); }
    __device__ static __forceinline__ uint32_t mnmajor_lo(uint32_t saddr) { return desc_lo(saddr, RT::SUB_BYTES); }
    // contraction block kb of an operand whose lower word is `lo`
    __device__ static __forceinline__ uint64_t kmajor(uint32_t lo, int kb) {
        return desc_join(lo + (kb >> 2) * static_cast<int>(RT::SUB_BYTES >> 4) + (kb & 3) * 2, HI);
    }
    __device__ static __forceinline__ uint64_t mnmajor(uint32_t lo, int kb) {
        return desc_join(lo + kb * static_cast<int>(RT::ROW_BYTES), HI);
    }
};

struct SqDesc {
    static constexpr uint32_t HI = desc_hi(1024, SWZ_128B);
    __device__ static __forceinline__ uint32_t kmajor_lo(uint32_t saddr) { return desc_lo(saddr, 16); }
    __device__ static __forceinline__ uint32_t mnmajor_lo(uint32_t saddr) { return desc_lo(saddr, SQ_SUB_BYTES); }
    __device__ static __forceinline__ uint64_t kmajor(uint32_t lo, int kb) {
        return desc_join(lo + (kb >> 2) * static_cast<int>(SQ_SUB_BYTES >> 4) + (kb & 3) * 2, HI);
    }
    __device__ static __forceinline__ uint64_t mnmajor(uint32_t lo, int kb) { return desc_join(lo + kb * 128, HI); }
};

}  // namespace evo
