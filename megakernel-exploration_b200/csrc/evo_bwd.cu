// EvoAttention backward for sm_100a.
//
// Replaces evo_bwd_prep_ker / evo_bwd_ker (evo_h100/tk_evoattention.cu:352-416,
// :613-890) and their host launcher (tk_evoattention.cu:1051-1197):
//
//   P  = exp(q k^T * scale + pair_bias + res_mask - LSE)      (recomputed)
//   dP = dO v^T,  dS = P o (dP - delta),  delta = rowsum(dO o O)
//   dV = P^T dO,  dK = scale * dS^T q,  dQ = scale * dS k
//   dBias[b,h,q,kv] = sum over s of dS        (unscaled, tk_evoattention.cu:824-833)
//
// Three launches on one stream:
//   1. bwd_prep_kernel   delta, -LSE*log2e and mask*log2e rows, padded to whole
//                        tiles so the main kernel needs no edge predicates
//   2. evo_bwd_kernel    the fused backward (below)
//   3. cvt_dq_kernel     fp32 dQ accumulator -> bf16 dQ in the caller layout
//
// evo_bwd_kernel: one persistent CTA per SM walks items (chunk of RC consecutive
// S rows, head h, kv tile j of 128 residues); per item it walks steps
// (q tile i, row r of the chunk), r innermost.  dK/dV of every row of the chunk
// stay in tensor memory for the whole item; dS of the RC rows that share one
// pair-bias tile is summed in registers before it is added to dBias, where the
// reference issues one scalar atomic per element per row
// (tk_evoattention.cu:583-611).
//
//   warp 8 (producer)  TMA: K/V tiles + mask rows per item; Q/dO tiles + LSE/delta
//                      rows per step; the pair-bias tile per q tile
//   warp 9 (mma)       tcgen05.mma: S = Q K^T, dP = dO V^T, then dV += P^T dO,
//                      dK += dS^T Q, dQ = dS K, accumulators in tensor memory
//   warps 0-3, 4-7     two compute groups; group g owns kv columns 64g..64g+63
//                      (thread = one q row): P, dS -> shared memory as bf16 MMA
//                      operands; dBias partial sums; drains dQ (TMA reduce-add
//                      into the fp32 accumulator), dBias (TMA reduce-add) and
//                      dK/dV (TMA store, bf16)
#include "evo_host.cuh"
#include "evo_tiles.cuh"

namespace evo {

constexpr int BWD_THREADS = 320;
constexpr int BWD_GROUP_THREADS = 256;
constexpr uint32_t BWD_TMEM_COLS = 512;

template <int DH>
struct BwdCfg {
    static constexpr int RC = (DH == 32) ? 2 : 1;    // S rows per chunk
    static constexpr int QS = (DH == 32) ? 2 : 1;    // Q/dO stages
    static constexpr int KVB = (DH == 32) ? 2 : 1;   // K/V buffers (items in flight)
    static constexpr uint32_t ROWT = RowTile<DH>::BYTES;
    static constexpr uint32_t OFF_K = 0;
    static constexpr uint32_t OFF_V = OFF_K + KVB * RC * ROWT;
    static constexpr uint32_t OFF_Q = OFF_V + KVB * RC * ROWT;
    static constexpr uint32_t OFF_DO = OFF_Q + QS * ROWT;
    static constexpr uint32_t OFF_BIAS = OFF_DO + QS * ROWT;
    static constexpr uint32_t OFF_P = OFF_BIAS + SQ_BYTES;
    static constexpr uint32_t OFF_DS = OFF_P + SQ_BYTES;          // P,dS contiguous: dBias staging
    static constexpr uint32_t OFF_DQS = OFF_DS + SQ_BYTES;        // fp32 [128][DH] dQ staging
    static constexpr uint32_t DQS_BYTES = 128 * DH * 4;
    static constexpr uint32_t OFF_ROWV = OFF_DQS + DQS_BYTES;     // per stage: nlse2[128], delta[128]
    static constexpr uint32_t OFF_MASK = OFF_ROWV + QS * 1024;    // [KVB][RC][128] float
    static constexpr uint32_t OFF_BARS = OFF_MASK + KVB * RC * 512;
    static constexpr uint32_t NUM_BARS = 2 * KVB + 2 * QS + 2 + 6 + 1;
    static constexpr uint32_t OFF_MISC = OFF_BARS + NUM_BARS * 8;
    static constexpr uint32_t SMEM_BYTES = OFF_MISC + 16 + 1024;  // + alignment slack
    static constexpr uint32_t TMEM_S = 0;
    static constexpr uint32_t TMEM_DP = 128;
    static constexpr uint32_t TMEM_DQ = 256;
    static constexpr uint32_t TMEM_DKV = 256 + DH;                // + r*2*DH (dK), + DH (dV)
    static_assert(TMEM_DKV + RC * 2 * DH <= BWD_TMEM_COLS, "tensor memory budget");
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct BwdParams {
    int B, S, N, H;
    int NT;          // tiles per row: ceil(N / 128)
    int NTP;         // NT * 128
    int CPB;         // chunks per batch: ceil(S / RC)
    int total_items; // B * CPB * H * NT
    float scale;     // softmax scale
    float c1;        // scale * log2(e)
    const float* nlse2;   // [B*S][H][NTP]  -LSE*log2e, -inf in the padding
    const float* delta;   // [B*S][H][NTP]  0 in the padding
    const float* maskl2;  // [B*S][NTP]     mask*log2e, -inf in the padding
    unsigned int* status;
};

struct BwdItem {
    int b, bs0, nr, h, j;
};

template <int DH>
__global__ void __launch_bounds__(BWD_THREADS, 1)
evo_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
               const __grid_constant__ CUtensorMap tm_bias, const __grid_constant__ CUtensorMap tm_dk,
               const __grid_constant__ CUtensorMap tm_dv, const __grid_constant__ CUtensorMap tm_dq,
               const __grid_constant__ CUtensorMap tm_dbias, const BwdParams p) {
    using C = BwdCfg<DH>;
    using RT = RowTile<DH>;
    constexpr int RC = C::RC, QS = C::QS, KVB = C::KVB;
    constexpr int HALF = DH / 2;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BARS);
    uint64_t* kv_full = bars;                  // [KVB]
    uint64_t* kv_empty = kv_full + KVB;        // [KVB]
    uint64_t* qd_full = kv_empty + KVB;        // [QS]
    uint64_t* qd_empty = qd_full + QS;         // [QS]
    uint64_t* bias_full = qd_empty + QS;
    uint64_t* bias_empty = bias_full + 1;
    uint64_t* sdp_full = bias_empty + 1;
    uint64_t* sdp_free = sdp_full + 1;
    uint64_t* pds_ready = sdp_free + 1;
    uint64_t* dq_full = pds_ready + 1;
    uint64_t* dq_free = dq_full + 1;
    uint64_t* dkv_free = dq_free + 1;
    uint64_t* grp_bar = dkv_free + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_MISC);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int NT = p.NT;
    WaitCtx wc{abort_flag, p.status};

    if (tid == 0) {
        *abort_flag = 0;
        for (int i = 0; i < KVB; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 9); }
        for (int i = 0; i < QS; ++i) { mbar_init(&qd_full[i], 1); mbar_init(&qd_empty[i], 9); }
        mbar_init(bias_full, 1);
        mbar_init(bias_empty, 8);
        mbar_init(sdp_full, 1);
        mbar_init(sdp_free, 8);
        mbar_init(pds_ready, 8);
        mbar_init(dq_full, 1);
        mbar_init(dq_free, 8);
        mbar_init(dkv_free, 8);
        mbar_init(grp_bar, BWD_GROUP_THREADS);
        fence_mbar_init();
        fence_async_smem();
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot, BWD_TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == 8 && lane == 0) {
        prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); prefetch_tmap(&tm_do);
        prefetch_tmap(&tm_bias); prefetch_tmap(&tm_dk); prefetch_tmap(&tm_dv); prefetch_tmap(&tm_dq);
        prefetch_tmap(&tm_dbias);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int first = blockIdx.x;
    const int stride = gridDim.x;
    const int n_items = (p.total_items > first) ? (p.total_items - first + stride - 1) / stride : 0;

    // item index -> (batch, first row, rows, head, kv tile); kv tile fastest, then head
    auto decode = [&](int it) -> BwdItem {
        BwdItem x;
        const int w = first + it * stride;
        x.j = w % NT;
        const int r1 = w / NT;
        x.h = r1 % p.H;
        const int r2 = r1 / p.H;
        const int c = r2 % p.CPB;
        x.b = r2 / p.CPB;
        const int s0 = c * RC;
        x.nr = (p.S - s0 < RC) ? (p.S - s0) : RC;
        x.bs0 = x.b * p.S + s0;
        return x;
    };

    if (warp == 8) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            bool ok = true;
            int gs = 0, gb = 0;
            for (int it = 0; it < n_items && ok; ++it) {
                const BwdItem x = decode(it);
                const int kb = it % KVB;
                if (it >= KVB) ok = mbar_wait(&kv_empty[kb], ((it / KVB) - 1) & 1, wc, 0x40);
                if (!ok) break;
                mbar_arrive_expect_tx(&kv_full[kb], x.nr * (2 * C::ROWT + 512));
                for (int r = 0; r < x.nr; ++r) {
                    const int t = kb * RC + r;
                    tma_load_4d(smem + C::OFF_K + t * C::ROWT, &tm_k, &kv_full[kb], 0, x.h, x.j * TILE, x.bs0 + r);
                    tma_load_4d(smem + C::OFF_V + t * C::ROWT, &tm_v, &kv_full[kb], 0, x.h, x.j * TILE, x.bs0 + r);
                    bulk_load(smem + C::OFF_MASK + t * 512,
                              p.maskl2 + static_cast<size_t>(x.bs0 + r) * p.NTP + x.j * TILE, 512, &kv_full[kb]);
                }
                const int nsteps = NT * x.nr;
                for (int n = 0; n < nsteps && ok; ++n, ++gs) {
                    const int i = n / x.nr, r = n - i * x.nr;
                    const int st = gs % QS;
                    if (r == 0) {
                        if (gb > 0) ok = mbar_wait(bias_empty, (gb - 1) & 1, wc, 0x41);
                        if (!ok) break;
                        mbar_arrive_expect_tx(bias_full, SQ_BYTES);
                        tma_load_4d(smem + C::OFF_BIAS, &tm_bias, bias_full, x.j * TILE, i * TILE, x.h, x.b);
                        tma_load_4d(smem + C::OFF_BIAS + SQ_SUB_BYTES, &tm_bias, bias_full, x.j * TILE + 64,
                                    i * TILE, x.h, x.b);
                        ++gb;
                    }
                    if (gs >= QS) ok = mbar_wait(&qd_empty[st], ((gs / QS) - 1) & 1, wc, 0x42);
                    if (!ok) break;
                    const int bs = x.bs0 + r;
                    mbar_arrive_expect_tx(&qd_full[st], 2 * C::ROWT + 1024);
                    tma_load_4d(smem + C::OFF_Q + st * C::ROWT, &tm_q, &qd_full[st], 0, x.h, i * TILE, bs);
                    tma_load_4d(smem + C::OFF_DO + st * C::ROWT, &tm_do, &qd_full[st], 0, x.h, i * TILE, bs);
                    const size_t ro = (static_cast<size_t>(bs) * p.H + x.h) * p.NTP + i * TILE;
                    bulk_load(smem + C::OFF_ROWV + st * 1024, p.nlse2 + ro, 512, &qd_full[st]);
                    bulk_load(smem + C::OFF_ROWV + st * 1024 + 512, p.delta + ro, 512, &qd_full[st]);
                }
            }
            // Drain: the most recent loads have landed before the CTA exits.
            for (int k = (gs > QS ? gs - QS : 0); k < gs; ++k)
                (void)mbar_wait(&qd_full[k % QS], (k / QS) & 1, wc, 0x43);
            if (gb > 0) (void)mbar_wait(bias_full, (gb - 1) & 1, wc, 0x44);
            for (int it = (n_items > KVB ? n_items - KVB : 0); it < n_items; ++it)
                (void)mbar_wait(&kv_full[it % KVB], (it / KVB) & 1, wc, 0x45);
        }
    } else if (warp == 9) {
        // ------------------------------ mma issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t IDESC_SDP = make_idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t IDESC_DKV = make_idesc_bf16(128, DH, 1, 1);
            constexpr uint32_t IDESC_DQ = make_idesc_bf16(128, DH, 0, 1);
            const uint32_t aK = smem_u32(smem + C::OFF_K), aV = smem_u32(smem + C::OFF_V);
            const uint32_t aQ = smem_u32(smem + C::OFF_Q), aDO = smem_u32(smem + C::OFF_DO);
            const uint32_t aP = smem_u32(smem + C::OFF_P), aDS = smem_u32(smem + C::OFF_DS);
            bool ok = true;

            // S and dP of step (it, n), global step gs
            auto issue_sdp = [&](int it, const BwdItem& x, int n, int gs) -> bool {
                const int kb = it % KVB, st = gs % QS;
                const int i = n / x.nr, r = n - i * x.nr;
                (void)i;
                if (n == 0 && !mbar_wait(&kv_full[kb], (it / KVB) & 1, wc, 0x50)) return false;
                if (!mbar_wait(&qd_full[st], (gs / QS) & 1, wc, 0x51)) return false;
                if (gs > 0 && !mbar_wait(sdp_free, (gs - 1) & 1, wc, 0x52)) return false;
                tc_fence_after();
                const uint32_t k_t = aK + (kb * RC + r) * C::ROWT, v_t = aV + (kb * RC + r) * C::ROWT;
#pragma unroll
                for (int kk = 0; kk < RT::KBLOCKS; ++kk)
                    umma_ss(tmem + C::TMEM_S, RT::kmajor(aQ + st * C::ROWT, kk), RT::kmajor(k_t, kk),
                            IDESC_SDP, kk > 0);
#pragma unroll
                for (int kk = 0; kk < RT::KBLOCKS; ++kk)
                    umma_ss(tmem + C::TMEM_DP, RT::kmajor(aDO + st * C::ROWT, kk), RT::kmajor(v_t, kk),
                            IDESC_SDP, kk > 0);
                umma_commit(sdp_full);
                return true;
            };
            // dV, dK, dQ of step (it, n)
            auto issue_tail = [&](int it, const BwdItem& x, int n, int gs) -> bool {
                const int kb = it % KVB, st = gs % QS;
                const int i = n / x.nr, r = n - i * x.nr;
                if (!mbar_wait(pds_ready, gs & 1, wc, 0x53)) return false;
                if (gs > 0 && !mbar_wait(dq_free, (gs - 1) & 1, wc, 0x54)) return false;
                if (n == 0 && it > 0 && !mbar_wait(dkv_free, (it - 1) & 1, wc, 0x55)) return false;
                tc_fence_after();
                const uint32_t k_t = aK + (kb * RC + r) * C::ROWT;
                const uint32_t q_t = aQ + st * C::ROWT, do_t = aDO + st * C::ROWT;
                const uint32_t t_dk = tmem + C::TMEM_DKV + r * 2 * DH, t_dv = t_dk + DH;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)
                    umma_ss(t_dv, sq_mnmajor(aP, kk), RT::mnmajor(do_t, kk), IDESC_DKV, (i > 0 || kk > 0));
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)
                    umma_ss(t_dk, sq_mnmajor(aDS, kk), RT::mnmajor(q_t, kk), IDESC_DKV, (i > 0 || kk > 0));
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)
                    umma_ss(tmem + C::TMEM_DQ, sq_kmajor(aDS, kk), RT::mnmajor(k_t, kk), IDESC_DQ, kk > 0);
                umma_commit(dq_full);
                umma_commit(&qd_empty[st]);
                if (n == NT * x.nr - 1) umma_commit(&kv_empty[kb]);
                return true;
            };

            int gs = 0;
            for (int it = 0; it < n_items && ok; ++it) {
                const BwdItem x = decode(it);
                const int nsteps = NT * x.nr;
                if (QS >= 2) {
                    // look one step ahead inside the item: S/dP of step n+1 are
                    // queued before dV/dK/dQ of step n
                    ok = issue_sdp(it, x, 0, gs);
                    for (int n = 0; n < nsteps && ok; ++n, ++gs) {
                        if (n + 1 < nsteps) ok = issue_sdp(it, x, n + 1, gs + 1);
                        if (ok) ok = issue_tail(it, x, n, gs);
                    }
                } else {
                    for (int n = 0; n < nsteps && ok; ++n, ++gs) {
                        ok = issue_sdp(it, x, n, gs);
                        if (ok) ok = issue_tail(it, x, n, gs);
                    }
                }
            }
        }
    } else {
        // ------------------------------ compute groups ------------------------------
        const int wg = warp >> 2;            // kv columns 64*wg .. 64*wg+63 of the tile
        const int row = tid & 127;           // q row within the tile == TMEM lane
        const int t256 = tid;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        uint8_t* sP = smem + C::OFF_P;
        uint8_t* sDS = smem + C::OFF_DS;
        uint8_t* sDQS = smem + C::OFF_DQS;
        bool ok = true;
        int gs = 0, gb = 0;
        uint32_t grp_phase = 0;
        auto group_sync = [&]() -> bool {
            mbar_arrive(grp_bar);
            const bool r = mbar_wait(grp_bar, grp_phase, wc, 0x60);
            grp_phase ^= 1u;
            return warp_all(r);
        };

        float acc[64];                       // dBias partial sums of this thread's 64 columns
        uint32_t bias_pk[32];                // this thread's 64 bias values (bf16 pairs)

        // Finishes step `pgs` (tile row pi of item px, chunk row pr): drains dQ into
        // the fp32 accumulator and, after the last row of the chunk, flushes dBias.
        auto finish_step = [&](const BwdItem& px, int pi, int pr, int pgs) -> bool {
            if (!warp_all(mbar_wait(dq_full, pgs & 1, wc, 0x61))) return false;
            tc_fence_after();
            float dq[HALF];
            tmem_ld_f32<HALF>(lane_base + C::TMEM_DQ + wg * HALF, dq);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(dq_free);
            const bool flush = (pr == px.nr - 1);
            // staging buffers are free once every earlier bulk reduce has read them
            if (t256 == 0) tma_wait_group_read<0>();
            if (!group_sync()) return false;
#pragma unroll
            for (int cc = 0; cc < HALF / 4; ++cc) {
                const int gc = wg * (HALF / 4) + cc;          // 16-byte chunk within the fp32 row
                const float4 v = make_float4(dq[cc * 4 + 0] * p.scale, dq[cc * 4 + 1] * p.scale,
                                             dq[cc * 4 + 2] * p.scale, dq[cc * 4 + 3] * p.scale);
                *reinterpret_cast<float4*>(sDQS + (gc >> 3) * 16384 + row * 128 + (((gc & 7) ^ (row & 7)) << 4)) = v;
            }
            if (flush) {
                // dBias staging over the (idle) P and dS tiles: four [128][32] fp32 boxes
#pragma unroll
                for (int cc = 0; cc < 16; ++cc) {
                    const int box = wg * 2 + (cc >> 3);
                    const float4 v = make_float4(acc[cc * 4 + 0], acc[cc * 4 + 1], acc[cc * 4 + 2], acc[cc * 4 + 3]);
                    *reinterpret_cast<float4*>(sP + box * 16384 + row * 128 + (((cc & 7) ^ (row & 7)) << 4)) = v;
                }
            }
            fence_async_smem();
            if (!group_sync()) return false;
            if (t256 == 0) {
#pragma unroll
                for (int bx = 0; bx < DH / 32; ++bx)
                    tma_reduce_add_4d(&tm_dq, sDQS + bx * 16384, bx * 32, px.h, pi * TILE, px.bs0 + pr);
                if (flush) {
                    for (int bx = 0; bx < 4; ++bx)
                        if (px.j * TILE + bx * 32 < p.N)
                            tma_reduce_add_4d(&tm_dbias, sP + bx * 16384, px.j * TILE + bx * 32, pi * TILE, px.h, px.b);
                }
                tma_commit_group();
                if (flush) tma_wait_group_read<0>();
            }
            if (flush) {
                // P / dS tiles are rewritten next: wait until the reduce has read them
                if (!group_sync()) return false;
            }
            return true;
        };

        for (int it = 0; it < n_items && ok; ++it) {
            const BwdItem x = decode(it);
            const int kb = it % KVB;
            const int nsteps = NT * x.nr;
            ok = warp_all(mbar_wait(&kv_full[kb], (it / KVB) & 1, wc, 0x62));   // mask rows
            if (!ok) break;
            for (int n = 0; n < nsteps && ok; ++n, ++gs) {
                const int i = n / x.nr, r = n - i * x.nr;
                const int st = gs % QS;
                ok = warp_all(mbar_wait(sdp_full, gs & 1, wc, 0x63));
                if (!ok) break;
                if (n > 0) {
                    const int pn = n - 1, pi = pn / x.nr, pr = pn - pi * x.nr;
                    ok = finish_step(x, pi, pr, gs - 1);
                    if (!ok) break;
                }
                if (r == 0) {
                    ok = warp_all(mbar_wait(bias_full, gb & 1, wc, 0x64));
                    if (!ok) break;
                    const uint8_t* sb = smem + C::OFF_BIAS + wg * SQ_SUB_BYTES + row * 128;
#pragma unroll
                    for (int c8 = 0; c8 < 8; ++c8) {
                        const uint4 bv = *reinterpret_cast<const uint4*>(sb + ((c8 ^ (row & 7)) << 4));
                        bias_pk[c8 * 4 + 0] = bv.x; bias_pk[c8 * 4 + 1] = bv.y;
                        bias_pk[c8 * 4 + 2] = bv.z; bias_pk[c8 * 4 + 3] = bv.w;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bias_empty);
                    ++gb;
#pragma unroll
                    for (int c = 0; c < 64; ++c) acc[c] = 0.f;
                }
                ok = warp_all(mbar_wait(&qd_full[st], (gs / QS) & 1, wc, 0x65));
                if (!ok) break;
                const float* rowv = reinterpret_cast<const float*>(smem + C::OFF_ROWV + st * 1024);
                const float nl = rowv[row];          // -LSE*log2e (-inf for padded rows)
                const float dl = rowv[128 + row];    // delta (0 for padded rows)
                __syncwarp();
                if (lane == 0) mbar_arrive(&qd_empty[st]);
                const float* mrow = reinterpret_cast<const float*>(smem + C::OFF_MASK + (kb * RC + r) * 512) + 64 * wg;

                tc_fence_after();
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    uint32_t sv[32], dv[32];
                    tmem_ld32(lane_base + C::TMEM_S + 64 * wg + 32 * hf, sv);
                    tmem_ld32(lane_base + C::TMEM_DP + 64 * wg + 32 * hf, dv);
                    tmem_wait_ld();
                    if (hf == 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(sdp_free);
                    }
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4) {
                        const float4 mv = *reinterpret_cast<const float4*>(mrow + 32 * hf + q4 * 4);
                        const float mm[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = q4 * 4 + e;                  // 0..31 within this half
                            const uint32_t word = bias_pk[hf * 16 + (c >> 1)];
                            const float bval = (c & 1) ? bf16_hi(word) : bf16_lo(word);
                            const float xv = fmaf(__uint_as_float(sv[c]), p.c1, fmaf(bval, LOG2E, mm[e]));
                            const float pv = ex2(xv + nl);
                            const float ds = pv * (__uint_as_float(dv[c]) - dl);
                            acc[hf * 32 + c] += ds;
                            sv[c] = __float_as_uint(pv);
                            dv[c] = __float_as_uint(ds);
                        }
                    }
#pragma unroll
                    for (int c8 = 0; c8 < 4; ++c8) {
                        uint4 v, w;
                        v.x = pack_bf16(__uint_as_float(sv[c8 * 8 + 0]), __uint_as_float(sv[c8 * 8 + 1]));
                        v.y = pack_bf16(__uint_as_float(sv[c8 * 8 + 2]), __uint_as_float(sv[c8 * 8 + 3]));
                        v.z = pack_bf16(__uint_as_float(sv[c8 * 8 + 4]), __uint_as_float(sv[c8 * 8 + 5]));
                        v.w = pack_bf16(__uint_as_float(sv[c8 * 8 + 6]), __uint_as_float(sv[c8 * 8 + 7]));
                        w.x = pack_bf16(__uint_as_float(dv[c8 * 8 + 0]), __uint_as_float(dv[c8 * 8 + 1]));
                        w.y = pack_bf16(__uint_as_float(dv[c8 * 8 + 2]), __uint_as_float(dv[c8 * 8 + 3]));
                        w.z = pack_bf16(__uint_as_float(dv[c8 * 8 + 4]), __uint_as_float(dv[c8 * 8 + 5]));
                        w.w = pack_bf16(__uint_as_float(dv[c8 * 8 + 6]), __uint_as_float(dv[c8 * 8 + 7]));
                        const uint32_t off = wg * SQ_SUB_BYTES + row * 128 + ((((hf * 4 + c8)) ^ (row & 7)) << 4);
                        *reinterpret_cast<uint4*>(sP + off) = v;
                        *reinterpret_cast<uint4*>(sDS + off) = w;
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(pds_ready);
            }
            if (!ok) break;
            // last step of the item
            {
                const int pn = nsteps - 1, pi = pn / x.nr, pr = pn - pi * x.nr;
                ok = finish_step(x, pi, pr, gs - 1);
                if (!ok) break;
            }
            if (lane == 0) mbar_arrive(&kv_empty[kb]);     // mask rows no longer needed

            // ---- dK / dV of every row of the chunk: tensor memory -> bf16 -> TMA store ----
            // staging: row tiles over the (idle) P tile, tile index 2*r (dK), 2*r+1 (dV)
            for (int r = 0; r < x.nr; ++r) {
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    float v[HALF];
                    tmem_ld_f32<HALF>(lane_base + C::TMEM_DKV + r * 2 * DH + t * DH + wg * HALF, v);
                    const float sc = (t == 0) ? p.scale : 1.0f;
                    uint8_t* dst = sP + (2 * r + t) * C::ROWT + row * RT::ROW_BYTES;
                    const int sw = (DH == 32) ? ((row >> 1) & 3) : (row & 7);
#pragma unroll
                    for (int c8 = 0; c8 < HALF / 8; ++c8) {
                        uint4 u;
                        u.x = pack_bf16(v[c8 * 8 + 0] * sc, v[c8 * 8 + 1] * sc);
                        u.y = pack_bf16(v[c8 * 8 + 2] * sc, v[c8 * 8 + 3] * sc);
                        u.z = pack_bf16(v[c8 * 8 + 4] * sc, v[c8 * 8 + 5] * sc);
                        u.w = pack_bf16(v[c8 * 8 + 6] * sc, v[c8 * 8 + 7] * sc);
                        const int chunk = wg * (HALF / 8) + c8;
                        *reinterpret_cast<uint4*>(dst + ((chunk ^ sw) << 4)) = u;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(dkv_free);
            fence_async_smem();
            ok = group_sync();
            if (!ok) break;
            if (t256 == 0) {
                for (int r = 0; r < x.nr; ++r) {
                    tma_store_4d(&tm_dk, sP + (2 * r) * C::ROWT, 0, x.h, x.j * TILE, x.bs0 + r);
                    tma_store_4d(&tm_dv, sP + (2 * r + 1) * C::ROWT, 0, x.h, x.j * TILE, x.bs0 + r);
                }
                tma_commit_group();
                tma_wait_group_read<0>();
            }
            ok = group_sync();           // the P tile may be rewritten
        }
        if (t256 == 0) tma_wait_group<0>();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem, BWD_TMEM_COLS);
}

// ---------------------------------------------------------------------------
// prep: delta = rowsum(dO o O) (replaces evo_bwd_prep_ker, tk_evoattention.cu:352-416),
// plus the pre-scaled, tile-padded LSE and mask rows the main kernel streams.
// ---------------------------------------------------------------------------
template <int DH>
__global__ void bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                const float* __restrict__ lse, const __nv_bfloat16* __restrict__ mask,
                                float* __restrict__ nlse2, float* __restrict__ delta,
                                float* __restrict__ maskl2, int BS, int N, int H, int NTP) {
    const size_t rows = static_cast<size_t>(BS) * N * H;
    const size_t gstride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const size_t t0 = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (size_t idx = t0; idx < rows; idx += gstride) {
        const int h = static_cast<int>(idx % H);
        const size_t bn = idx / H;
        const int n = static_cast<int>(bn % N);
        const size_t bs = bn / N;
        const uint4* po = reinterpret_cast<const uint4*>(o + idx * DH);
        const uint4* pd = reinterpret_cast<const uint4*>(d_o + idx * DH);
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < DH / 8; ++c) {
            const uint4 a = po[c], b = pd[c];
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s = fmaf(bf16_lo(aw[e]), bf16_lo(bw[e]), s);
                s = fmaf(bf16_hi(aw[e]), bf16_hi(bw[e]), s);
            }
        }
        const size_t ro = (bs * H + h) * NTP + n;
        delta[ro] = s;
        nlse2[ro] = -lse[(bs * H + h) * N + n] * LOG2E;
    }
    // padding of the row vectors, and the mask rows
    const int pad = NTP - N;
    const size_t npad = static_cast<size_t>(BS) * H * pad;
    for (size_t idx = t0; idx < npad; idx += gstride) {
        const size_t bh = idx / pad;
        const int n = N + static_cast<int>(idx % pad);
        delta[bh * NTP + n] = 0.f;
        nlse2[bh * NTP + n] = -INFINITY;
    }
    const size_t nmask = static_cast<size_t>(BS) * NTP;
    for (size_t idx = t0; idx < nmask; idx += gstride) {
        const size_t bs = idx / NTP;
        const int n = static_cast<int>(idx % NTP);
        maskl2[idx] = (n < N) ? __bfloat162float(mask[bs * N + n]) * LOG2E : -INFINITY;
    }
}

// fp32 accumulator -> bf16, 8 elements per thread
__global__ void cvt_dq_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n8) {
    const size_t gstride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += gstride) {
        const float4 a = reinterpret_cast<const float4*>(src)[2 * i];
        const float4 b = reinterpret_cast<const float4*>(src)[2 * i + 1];
        uint4 u;
        u.x = pack_bf16(a.x, a.y); u.y = pack_bf16(a.z, a.w);
        u.z = pack_bf16(b.x, b.y); u.w = pack_bf16(b.z, b.w);
        reinterpret_cast<uint4*>(dst)[i] = u;
    }
}

struct BwdWorkspace {
    size_t off_nlse2, off_delta, off_maskl2, off_dq, total;
};

static BwdWorkspace bwd_workspace(const EvoDims* d) {
    const size_t BS = static_cast<size_t>(d->B) * d->S;
    const size_t NTP = static_cast<size_t>((d->N + TILE - 1) / TILE) * TILE;
    auto up = [](size_t x) { return (x + 255) & ~static_cast<size_t>(255); };
    BwdWorkspace w;
    w.off_nlse2 = 0;
    w.off_delta = up(w.off_nlse2 + BS * d->H * NTP * 4);
    w.off_maskl2 = up(w.off_delta + BS * d->H * NTP * 4);
    w.off_dq = up(w.off_maskl2 + BS * NTP * 4);
    w.total = up(w.off_dq + BS * d->N * d->H * d->D * 4);
    return w;
}

template <int DH>
static int launch_bwd(const EvoDims* d, const void* q, const void* k, const void* v, const void* bias,
                      const void* mask, const void* o, const float* lse, const void* d_o, void* dq,
                      void* dk, void* dv, float* dbias, uint8_t* ws, float scale, cudaStream_t st) {
    using C = BwdCfg<DH>;
    const int BS = d->B * d->S;
    const int NT = (d->N + TILE - 1) / TILE;
    const BwdWorkspace w = bwd_workspace(d);
    float* nlse2 = reinterpret_cast<float*>(ws + w.off_nlse2);
    float* delta = reinterpret_cast<float*>(ws + w.off_delta);
    float* maskl2 = reinterpret_cast<float*>(ws + w.off_maskl2);
    float* dq_acc = reinterpret_cast<float*>(ws + w.off_dq);

    CUtensorMap tq, tk, tv, tdo, tb, tdk, tdv, tdq, tdb;
    int rc;
    if ((rc = make_tmap_qkv(&tq, q, BS, d->N, d->H, DH, TILE))) return rc;
    if ((rc = make_tmap_qkv(&tk, k, BS, d->N, d->H, DH, TILE))) return rc;
    if ((rc = make_tmap_qkv(&tv, v, BS, d->N, d->H, DH, TILE))) return rc;
    if ((rc = make_tmap_qkv(&tdo, d_o, BS, d->N, d->H, DH, TILE))) return rc;
    if ((rc = make_tmap_bias(&tb, bias, d->B, d->H, d->N))) return rc;
    if ((rc = make_tmap_qkv(&tdk, dk, BS, d->N, d->H, DH, TILE))) return rc;
    if ((rc = make_tmap_qkv(&tdv, dv, BS, d->N, d->H, DH, TILE))) return rc;
    if ((rc = make_tmap_qkv_f32(&tdq, dq_acc, BS, d->N, d->H, DH, TILE))) return rc;
    if ((rc = make_tmap_dbias(&tdb, dbias, d->B, d->H, d->N))) return rc;

    BwdParams p;
    p.B = d->B; p.S = d->S; p.N = d->N; p.H = d->H;
    p.NT = NT;
    p.NTP = NT * TILE;
    p.CPB = (d->S + C::RC - 1) / C::RC;
    p.total_items = d->B * p.CPB * d->H * NT;
    p.scale = (scale > 0.f) ? scale : 1.0f / sqrtf(static_cast<float>(DH));
    p.c1 = p.scale * LOG2E;
    p.nlse2 = nlse2; p.delta = delta; p.maskl2 = maskl2;
    p.status = status_word();
    if (!p.status) return EVO_ERR_CUDA;

    int dev = 0, sms = 0;
    if ((rc = cuda_err(cudaGetDevice(&dev)))) return rc;
    if ((rc = cuda_err(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)))) return rc;

    const size_t dq_bytes = static_cast<size_t>(BS) * d->N * d->H * DH * 4;
    const size_t db_bytes = static_cast<size_t>(d->B) * d->H * d->N * d->N * 4;
    if ((rc = cuda_err(cudaMemsetAsync(dq_acc, 0, dq_bytes, st)))) return rc;
    if ((rc = cuda_err(cudaMemsetAsync(dbias, 0, db_bytes, st)))) return rc;

    bwd_prep_kernel<DH><<<sms * 8, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), lse,
        static_cast<const __nv_bfloat16*>(mask), nlse2, delta, maskl2, BS, d->N, d->H, p.NTP);
    if ((rc = cuda_err(cudaGetLastError()))) return rc;

    if ((rc = cuda_err(cudaFuncSetAttribute(evo_bwd_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(C::SMEM_BYTES)))))
        return rc;
    const int grid = p.total_items < sms ? p.total_items : sms;
    evo_bwd_kernel<DH><<<grid, BWD_THREADS, C::SMEM_BYTES, st>>>(tq, tk, tv, tdo, tb, tdk, tdv, tdq, tdb, p);
    if ((rc = cuda_err(cudaGetLastError()))) return rc;

    cvt_dq_kernel<<<sms * 8, 256, 0, st>>>(dq_acc, static_cast<__nv_bfloat16*>(dq), dq_bytes / 32);
    return cuda_err(cudaGetLastError());
}

}  // namespace evo

extern "C" size_t evo_bwd_workspace_bytes(const EvoDims* dims) {
    if (evo::check_dims(dims) != EVO_OK) return 0;
    return evo::bwd_workspace(dims).total;
}

extern "C" int evo_bwd(const EvoDims* dims, const void* q, const void* k, const void* v,
                       const void* pair_bias, const void* res_mask, const void* o, const float* lse,
                       const void* d_o, void* dq, void* dk, void* dv, float* dbias, void* workspace,
                       size_t workspace_bytes, float scale, void* stream) {
    int rc = evo::check_dims(dims);
    if (rc) return rc;
    if (!q || !k || !v || !pair_bias || !res_mask || !o || !lse || !d_o || !dq || !dk || !dv || !dbias ||
        !workspace)
        return EVO_ERR_NULL_PTR;
    const uintptr_t all = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                          reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(pair_bias) |
                          reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(d_o) |
                          reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) |
                          reinterpret_cast<uintptr_t>(dv) | reinterpret_cast<uintptr_t>(dbias) |
                          reinterpret_cast<uintptr_t>(lse);
    if (all & 15u) return EVO_ERR_ALIGNMENT;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < evo::bwd_workspace(dims).total)
        return EVO_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    if (dims->D == 32)
        return evo::launch_bwd<32>(dims, q, k, v, pair_bias, res_mask, o, lse, d_o, dq, dk, dv, dbias, ws, scale, st);
    return evo::launch_bwd<64>(dims, q, k, v, pair_bias, res_mask, o, lse, d_o, dq, dk, dv, dbias, ws, scale, st);
}
