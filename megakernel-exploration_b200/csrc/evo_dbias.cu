// Pair-bias gradient for sm_100a.
//
//   dBias[b,h,i,j] = sum_s dS[b,s,h,i,j],   dS = P o (dP - delta),
//   P = exp(scale * Q K^T + bias + mask - LSE),   dP = dO V^T
//
// The reference accumulates this sum with fp32 atomics from inside its backward
// kernel (evo_h100/tk_evoattention.cu:806-813 in bwd_attend_ker).  Here the sum
// is turned inside out: a CTA owns one [128 x 128] tile of the pair bias for a
// slice of the S rows and keeps the running sum in registers, so the only
// traffic of the reduction is one write (or one vector atomic per slice) of the
// finished tile.  S and dP are recomputed for that (the dQ/dK/dV kernel computes
// them too); the recompute costs two small MMAs per step, and the elementwise
// work runs without the shared-memory round trips the dQ/dK/dV kernel needs
// for its operands.
//
//   warp NCW   (producer)  TMA per step (one S row): Q, dO tiles of q tile i,
//                          K, V tiles of kv tile j, and the two extra tiles of the
//                          step (per-row terms of i, per-column terms of j)
//   warp NCW+1 (mma)       S' = Q K^T + (mask - LSE) / scale and dP' = dO V^T - delta
//                          into one of two tensor memory buffers, so the MMAs of
//                          step n+1 overlap the elementwise work of step n.  The
//                          additive terms ride in an extra contraction block
//                          (evo_tiles.cuh), so the elementwise work is one fused
//                          multiply-add, one exp2 and one accumulate per element
//   warps 0..NCW-1         NG compute groups of four warps; group g owns kv
//                          columns g*CW .. g*CW+CW-1 of the tile, thread = q row.
//                          Bias (bf16 pairs) and the running sum stay in
//                          registers for the whole item.
#include "evo_dbias.cuh"
#include "evo_host.cuh"
#include "evo_ptx.cuh"
#include "evo_tiles.cuh"

namespace evo {

// every fourth column pair takes its exp2 on the fused-multiply-add pipe (see ex2_poly2)
#ifndef EVO_DBIAS_POLY_EVERY
#define EVO_DBIAS_POLY_EVERY 4
#endif
constexpr int DBIAS_POLY_EVERY = EVO_DBIAS_POLY_EVERY;

template <int DH, int NG>
struct DbCfg {
    static constexpr int CW = TILE / NG;                  // kv columns per thread
    static constexpr int NCW = NG * 4;                    // compute warps
    static constexpr int THREADS = (NCW + 4) * 32;        // + one warpgroup: producer, mma, two idle warps
    // setmaxnreg budgets.  The CTA's register pool is what it was launched with
    // (the per-thread cap ptxas derives from the launch bound, times THREADS); an
    // increase blocks until the pool has room, for ever if it never can.
    static constexpr int REGS_LAUNCH = (65536 / THREADS) & ~7;
    // measured (B=1, S=512, N=384, H=8, D=32 / B=1, S=256, N=1024, H=4, D=64): 224/56 0.200 / 0.394 ms,
    // 216/72 0.195 / 0.380, 208/88 0.213 / 0.409
    static constexpr int REGS_COMPUTE = (NG == 2) ? 216 : 112;
    static constexpr int REGS_OTHER = (NG == 2) ? 72 : 32;
    static_assert(REGS_COMPUTE * NCW * 32 + REGS_OTHER * 128 <= REGS_LAUNCH * THREADS, "register pool");
    // D <= 64: a stage holds the four operand tiles of a step.  D = 128 (four tiles are 128 KB):
    // a stage holds ONE operand pair, (Q, K) of a step or (dO, V) of a step, alternately; each of
    // the two issuer warps issues from its own pair and both release every stage.
    static constexpr int SPLIT = (DH == 128) ? 2 : 1;     // stages per step
    static constexpr int QS = (DH == 32) ? 6 : 3;         // load stages
    static constexpr uint32_t ROWT = RowTile<DH>::BYTES;
    static constexpr uint32_t ST_Q = 0, ST_DO = (SPLIT == 2) ? 0 : ROWT;
    static constexpr uint32_t ST_K = (SPLIT == 2) ? ROWT : 2 * ROWT, ST_V = (SPLIT == 2) ? ROWT : 3 * ROWT;
    static constexpr uint32_t ST_XQ = (4 / SPLIT) * ROWT, ST_XK = ST_XQ + XT_BYTES;     // extra tiles of the step
    static constexpr uint32_t STAGE_TX = 4 * ROWT + 2 * XT_BYTES;            // SPLIT == 1
    static constexpr uint32_t STAGE_STRIDE = (4 / SPLIT) * ROWT + 2 * XT_BYTES;
    // constant extra tiles, above every stage (the zero tile must sit above the tiles that refer to it)
    static constexpr uint32_t OFF_XDP = QS * STAGE_STRIDE;                    // column selector of -delta
    static constexpr uint32_t OFF_ZERO = OFF_XDP + XT_BYTES;
    static constexpr uint32_t OFF_BARS = OFF_ZERO + XT_BYTES;
    static constexpr uint32_t NUM_BARS = 2 * QS + 4;
    static constexpr uint32_t OFF_MISC = OFF_BARS + NUM_BARS * 8;
    static constexpr uint32_t SMEM_BYTES = OFF_MISC + 16 + 1024;
    static constexpr uint32_t TMEM_COLS = 512;            // two buffers of S[128] | dP[128]
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
    static_assert(CW % 16 == 0, "columns per thread");
};

struct DbParams {
    int B, S, N, H;
    int NT, NTP;
    int KB;               // contraction blocks of 16 head-dim columns that hold data: ceil(D / 16)
    int Z, SL;            // S slices, rows per slice
    int total_items;      // Z * B * H * NT * NT
    float c1;             // scale * log2(e)
    const __nv_bfloat16* xq;     // [B*S][H][NTP][8] extra tiles: per-row terms (see bwd_prep_kernel)
    const __nv_bfloat16* xk;     // [B*S][NTP][8]    extra tiles: per-column terms
    const __nv_bfloat16* bias;   // [B][H][N][N]
    float* dbias;                // [B][H][N][N]
    unsigned int* status;
};

struct DbItem {
    int b, h, i, j, s0, ns;
};

template <int DH, int NG>
__global__ void __launch_bounds__(DbCfg<DH, NG>::THREADS, 1)
evo_dbias_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                 const DbParams p) {
    using C = DbCfg<DH, NG>;
    using RT = RowTile<DH>;
    using RD = RowDesc<DH>;
    constexpr int QS = C::QS, CW = C::CW, NCW = C::NCW;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BARS);
    uint64_t* st_full = bars;                 // [QS]
    uint64_t* st_empty = st_full + QS;        // [QS]
    uint64_t* sdp_full = st_empty + QS;       // [2]
    uint64_t* sdp_free = sdp_full + 2;        // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_MISC);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int NT = p.NT;
    WaitCtx wc{abort_flag, p.status};

    if (tid == 0) {
        *abort_flag = 0;
        for (int i = 0; i < QS; ++i) { mbar_init(&st_full[i], 1); mbar_init(&st_empty[i], 2); }
        for (int i = 0; i < 2; ++i) { mbar_init(&sdp_full[i], 2); mbar_init(&sdp_free[i], NCW); }
        fence_mbar_init();
        fence_async_smem();
    }
    if (warp == NCW + 1) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == NCW && lane == 0) {
        prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); prefetch_tmap(&tm_do);
    }
    // constant extra tiles: row n of the -delta selector is (0,0,0,0,1,1,0,0); the zero tile
    for (int r = tid; r < 128; r += C::THREADS) {
        *reinterpret_cast<uint4*>(smem + C::OFF_XDP + r * 16) = make_uint4(0u, 0u, 0x3f803f80u, 0u);
        *reinterpret_cast<uint4*>(smem + C::OFF_ZERO + r * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    fence_async_smem();
    EVO_TRACE_INIT();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    EVO_TS(t_kernel);

    const int first = blockIdx.x;
    const int stride = gridDim.x;
    const int n_items = (p.total_items > first) ? (p.total_items - first + stride - 1) / stride : 0;

    // item index -> (slice, batch, head, q tile, kv tile); kv tile fastest, so CTAs
    // that run side by side read the same S rows of the same head
    auto decode = [&](int it) -> DbItem {
        DbItem x;
        int w = first + it * stride;
        x.j = w % NT; w /= NT;
        x.i = w % NT; w /= NT;
        x.h = w % p.H; w /= p.H;
        x.b = w % p.B; w /= p.B;
        x.s0 = w * p.SL;
        x.ns = (p.S - x.s0 < p.SL) ? (p.S - x.s0) : p.SL;
        return x;
    };

    if (warp >= NCW) {
        reg_dec<C::REGS_OTHER>();
        if (warp == NCW) {
            if (lane == 0) {
                // ------------------------------ producer ------------------------------
                bool ok = true;
                int gs = 0;
                for (int it = 0; it < n_items && ok; ++it) {
                    const DbItem x = decode(it);
                    for (int n = 0; n < x.ns && ok; ++n, ++gs) {
                        const int bs = x.b * p.S + x.s0 + n;
                        const size_t ro = (static_cast<size_t>(bs) * p.H + x.h) * p.NTP + x.i * TILE;
#pragma unroll
                        for (int hf = 0; hf < C::SPLIT; ++hf) {
                            const int ld = gs * C::SPLIT + hf;        // running load counter
                            const int st = ld % QS;
                            if (ld >= QS) ok = mbar_wait(&st_empty[st], ((ld / QS) - 1) & 1, wc, 0x82);
                            if (!ok) break;
                            uint8_t* sb = smem + st * C::STAGE_STRIDE;
                            const bool with_s = (C::SPLIT == 1 || hf == 0), with_dp = (C::SPLIT == 1 || hf == 1);
                            mbar_arrive_expect_tx(&st_full[st], C::SPLIT == 1 ? C::STAGE_TX
                                                                             : 2 * C::ROWT + (hf == 0 ? 2 : 1) * XT_BYTES);
                            if (with_s) {
                                tma_load_row_tile<DH>(sb + C::ST_Q, &tm_q, &st_full[st], x.h, x.i * TILE, bs);
                                tma_load_row_tile<DH>(sb + C::ST_K, &tm_k, &st_full[st], x.h, x.j * TILE, bs);
                                bulk_load(sb + C::ST_XK, p.xk + (static_cast<size_t>(bs) * p.NTP + x.j * TILE) * 8,
                                          XT_BYTES, &st_full[st]);
                            }
                            if (with_dp) {
                                tma_load_row_tile<DH>(sb + C::ST_DO, &tm_do, &st_full[st], x.h, x.i * TILE, bs);
                                tma_load_row_tile<DH>(sb + C::ST_V, &tm_v, &st_full[st], x.h, x.j * TILE, bs);
                            }
                            bulk_load(sb + C::ST_XQ, p.xq + ro * 8, XT_BYTES, &st_full[st]);
                        }
                    }
                }
                // the most recent loads have landed before the CTA exits
                const int loads = gs * C::SPLIT;
                for (int k = (loads > QS ? loads - QS : 0); k < loads; ++k)
                    (void)mbar_wait(&st_full[k % QS], (k / QS) & 1, wc, 0x83);
            }
        } else if (warp == NCW + 1 || warp == NCW + 2) {
            // ------------------------------ mma issuers ------------------------------
            // warp NCW+1 issues S' = Q K^T + extra block, warp NCW+2 issues dP' = dO V^T + extra
            // block, so that neither chain queues behind the other's issue.  Each warp runs its
            // loop with all lanes (uniform control flow keeps the operand descriptors in uniform
            // registers) and elects one lane to issue.
            constexpr uint32_t IDESC = make_idesc_bf16(128, 128, 0, 0);
            const bool is_dp = (warp == NCW + 2);
            const uint32_t aSt = smem_u32(smem);
            const uint32_t aZero = aSt + C::OFF_ZERO;
            bool ok = true;
            int gs = 0;
            for (int it = 0; it < n_items && ok; ++it) {
                const DbItem x = decode(it);
                for (int n = 0; n < x.ns && ok; ++n, ++gs) {
                    const int ld = gs * C::SPLIT + ((C::SPLIT == 2 && is_dp) ? 1 : 0);
                    const int st = ld % QS, buf = gs & 1;
                    if (C::SPLIT == 2) {
                        // The other issuer's stage of this step: observed and released unused, in load
                        // order.  A parity wait tells "this phase is over" only to a waiter that saw
                        // the previous phase end; a warp that skipped the other warp's uses of a stage
                        // could take a load that has not landed yet for its own, two uses later.
                        const int lo = gs * 2 + (is_dp ? 0 : 1);
                        if (is_dp) {
                            ok = warp_all(mbar_wait(&st_full[lo % QS], (lo / QS) & 1, wc, 0x92));
                            if (ok && elect_one()) mbar_arrive(&st_empty[lo % QS]);
                            __syncwarp();
                        }
                    }
                    if (ok) ok = warp_all(mbar_wait(&st_full[st], (ld / QS) & 1, wc, 0x90));
                    if (ok && gs >= 2) ok = warp_all(mbar_wait(&sdp_free[buf], ((gs >> 1) - 1) & 1, wc, 0x91));
                    if (!ok) break;
                    tc_fence_after();
                    if (elect_one()) {
                        const uint32_t sb = aSt + st * C::STAGE_STRIDE;
                        const uint32_t t0 = tmem + buf * 256 + (is_dp ? 128u : 0u);
                        const uint32_t a_lo = RD::kmajor_lo(sb + (is_dp ? C::ST_DO : C::ST_Q));
                        const uint32_t b_lo = RD::kmajor_lo(sb + (is_dp ? C::ST_V : C::ST_K));
#pragma unroll
                        for (int kk = 0; kk < RT::KBLOCKS; ++kk)
                            if (kk < p.KB)      // blocks past the true head dim are zero-filled: skipped
                                umma_ss(t0, RD::kmajor(a_lo, kk), RD::kmajor(b_lo, kk), IDESC, kk > 0);
                        // + (mask - LSE) / scale on S, - delta on dP: the extra contraction block
                        umma_ss(t0, xt_desc(sb + C::ST_XQ, aZero),
                                xt_desc(is_dp ? aSt + C::OFF_XDP : sb + C::ST_XK, aZero), IDESC, 1u);
                        umma_commit(&sdp_full[buf]);
                        umma_commit(&st_empty[st]);
                    }
                    __syncwarp();
                    if (C::SPLIT == 2 && !is_dp) {
                        const int lo = gs * 2 + 1;
                        ok = warp_all(mbar_wait(&st_full[lo % QS], (lo / QS) & 1, wc, 0x92));
                        if (ok && elect_one()) mbar_arrive(&st_empty[lo % QS]);
                        __syncwarp();
                    }
                }
            }
        }
    } else {
        reg_inc<C::REGS_COMPUTE>();
        // ------------------------------ compute groups ------------------------------
        const int g = warp >> 2;                   // kv columns g*CW .. of the tile
        const int wrow0 = (warp & 3) * 32;
        const int row = wrow0 + lane;              // q row within the tile == TMEM lane
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(wrow0) << 16) + g * CW;
        bool ok = true;
        int gs = 0;
        const float2 c1x2 = make_float2(p.c1, p.c1);

        for (int it = 0; it < n_items && ok; ++it) {
            const DbItem x = decode(it);
            const int qrow = x.i * TILE + row;
            const int col0 = x.j * TILE + g * CW;
            const size_t tile_off = ((static_cast<size_t>(x.b) * p.H + x.h) * p.N + qrow) * p.N + col0;

            // this thread's CW bias values, times log2(e), and the running sums: registers for the item
            float2 bl2[CW / 2], acc[CW / 2];
#pragma unroll
            for (int c8 = 0; c8 < CW / 8; ++c8) {
                uint4 bv = make_uint4(0u, 0u, 0u, 0u);
                if (qrow < p.N && col0 + c8 * 8 < p.N)
                    bv = __ldg(reinterpret_cast<const uint4*>(p.bias + tile_off + c8 * 8));
                const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = bf16x2_f2(bw[e]);
                    bl2[c8 * 4 + e] = make_float2(f.x * LOG2E, f.y * LOG2E);
                }
            }
#pragma unroll
            for (int c = 0; c < CW / 2; ++c) acc[c] = make_float2(0.f, 0.f);

            for (int n = 0; n < x.ns && ok; ++n, ++gs) {
                const int buf = gs & 1;
                ok = warp_all(mbar_wait(&sdp_full[buf], (gs >> 1) & 1, wc, 0xa0));
                if (!ok) break;
                EVO_TS(t_math);
                tc_fence_after();
                // Chunks of 16 columns.  The tensor-memory loads of chunk ch+1 are in flight
                // during the arithmetic of chunk ch.  Per element: x = S' c1 + bias log2e (S'
                // already carries mask and -LSE), P = exp2(x), sum += P dP' (dP' already
                // carries -delta).
                uint32_t sv[2][16], dv[2][16];
                tmem_ld16(lane_base + buf * 256, sv[0]);
                tmem_ld16(lane_base + buf * 256 + 128, dv[0]);
#pragma unroll
                for (int ch = 0; ch < CW / 16; ++ch) {
                    const int cb = ch & 1;
                    tmem_wait_ld();
                    if (ch + 1 < CW / 16) {
                        tmem_ld16(lane_base + buf * 256 + 16 * (ch + 1), sv[cb ^ 1]);
                        tmem_ld16(lane_base + buf * 256 + 128 + 16 * (ch + 1), dv[cb ^ 1]);
                    } else {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&sdp_free[buf]);
                    }
                    float2 p2[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const float2 x2 = ffma2(u2f2(sv[cb][2 * k], sv[cb][2 * k + 1]), c1x2, bl2[ch * 8 + k]);
                        p2[k] = use_poly<DBIAS_POLY_EVERY>(k) ? ex2_poly2(x2) : make_float2(ex2(x2.x), ex2(x2.y));
                    }
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        acc[ch * 8 + k] = ffma2(p2[k], u2f2(dv[cb][2 * k], dv[cb][2 * k + 1]), acc[ch * 8 + k]);
                }
                EVO_TE(t_math, p.status, 0xa8);
            }
            if (!ok) break;

            // the finished tile: plain stores when this CTA saw every S row, else atomics
            if (qrow < p.N) {
                float* out = p.dbias + tile_off;
#pragma unroll
                for (int c4 = 0; c4 < CW / 4; ++c4) {
                    if (col0 + c4 * 4 < p.N) {
                        if (p.Z == 1) {
                            *reinterpret_cast<float4*>(out + c4 * 4) =
                                make_float4(acc[c4 * 2].x, acc[c4 * 2].y, acc[c4 * 2 + 1].x, acc[c4 * 2 + 1].y);
                        } else {
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + c4 * 4),
                                         "f"(acc[c4 * 2].x), "f"(acc[c4 * 2].y), "f"(acc[c4 * 2 + 1].x),
                                         "f"(acc[c4 * 2 + 1].y)
                                         : "memory");
                        }
                    }
                }
            }
        }
    }

    if (tid == 0) EVO_TE(t_kernel, p.status, 0xaf);
    tc_fence_before();
    __syncthreads();
    EVO_TRACE_FLUSH(p.status);
    if (warp == NCW + 1) tmem_dealloc(tmem, C::TMEM_COLS);
}

#ifndef EVO_DBIAS_GROUPS
#define EVO_DBIAS_GROUPS 2
#endif

template <int DH>
static int launch_dbias_t(const EvoDims* d, const ActLayout& lay, const ActLayout& lay_do, const void* q, const void* k, const void* v, const void* bias,
                          const void* d_o, const void* xq, const void* xk,
                          float* dbias, float scale, int sms, cudaStream_t st) {
    constexpr int NG = EVO_DBIAS_GROUPS;
    using C = DbCfg<DH, NG>;
    const int BS = d->B * d->S;
    const int NT = (d->N + TILE - 1) / TILE;

    CUtensorMap tq, tk, tv, tdo;
    int rc;
    if ((rc = make_tmap_qkv(&tq, q, BS, d->N, d->H, d->D, TILE, lay, RowTile<DH>::BOX_D))) return rc;
    if ((rc = make_tmap_qkv(&tk, k, BS, d->N, d->H, d->D, TILE, lay, RowTile<DH>::BOX_D))) return rc;
    if ((rc = make_tmap_qkv(&tv, v, BS, d->N, d->H, d->D, TILE, lay, RowTile<DH>::BOX_D))) return rc;
    if ((rc = make_tmap_qkv(&tdo, d_o, BS, d->N, d->H, d->D, TILE, lay_do, RowTile<DH>::BOX_D))) return rc;

    // Slices of S: enough items to fill the SMs evenly, each long enough that the
    // per-item set-up (bias load, pipeline fill, tile write) stays small.
    const long base = static_cast<long>(d->B) * d->H * NT * NT;
    int best_z = 1;
    long best_cost = -1;
    const int zmax = d->S < 64 ? d->S : 64;
    for (int z = 1; z <= zmax; ++z) {
        const int sl = (d->S + z - 1) / z;
        const int zz = (d->S + sl - 1) / sl;
        const long waves = (base * zz + sms - 1) / sms;
        const long cost = waves * (sl + 6);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_z = zz; }
    }

    DbParams p;
    p.B = d->B; p.S = d->S; p.N = d->N; p.H = d->H;
    p.NT = NT; p.NTP = NT * TILE;
    p.KB = (d->D + 15) / 16;
    p.SL = (d->S + best_z - 1) / best_z;
    p.Z = (d->S + p.SL - 1) / p.SL;
    p.total_items = static_cast<int>(base * p.Z);
    const float sc = (scale > 0.f) ? scale : 1.0f / sqrtf(static_cast<float>(d->D));
    p.c1 = sc * LOG2E;
    p.xq = static_cast<const __nv_bfloat16*>(xq);
    p.xk = static_cast<const __nv_bfloat16*>(xk);
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.dbias = dbias;
    p.status = status_word();
    if (!p.status) return EVO_ERR_CUDA;

    if ((rc = set_max_smem_once(reinterpret_cast<const void*>(evo_dbias_kernel<DH, NG>),
                                static_cast<int>(C::SMEM_BYTES))))
        return rc;
    const int grid = p.total_items < sms ? p.total_items : sms;
    prof_begin(2, st);
    evo_dbias_kernel<DH, NG><<<grid, C::THREADS, C::SMEM_BYTES, st>>>(tq, tk, tv, tdo, p);
    prof_end(2, st);
    return cuda_err(cudaGetLastError());
}

int launch_dbias(const EvoDims* d, const ActLayout& lay, const ActLayout& lay_do, const void* q, const void* k, const void* v, const void* bias,
                 const void* d_o, const void* xq, const void* xk, float* dbias,
                 float scale, int sms, cudaStream_t st) {
    if (d->D <= 32)
        return launch_dbias_t<32>(d, lay, lay_do, q, k, v, bias, d_o, xq, xk, dbias, scale, sms, st);
    if (d->D <= 64)
        return launch_dbias_t<64>(d, lay, lay_do, q, k, v, bias, d_o, xq, xk, dbias, scale, sms, st);
    return launch_dbias_t<128>(d, lay, lay_do, q, k, v, bias, d_o, xq, xk, dbias, scale, sms, st);
}

}  // namespace evo
