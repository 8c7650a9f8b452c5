// EvoAttention forward for sm_100a.
//
//   O = softmax(q k^T * scale + pair_bias + res_mask) v      per (b, s, h)
//
// replaces evo_fwd_ker (evo_h100/tk_evoattention.cu:102-345) and its host
// launcher (tk_evoattention.cu:911-1043).  Reads q/k/v and writes O directly in
// the caller layout [B][S][N][H][D] through strided TMA tensor maps: no
// transposes, no head-dim padding.
//
// One persistent CTA per SM walks work items (b*s, q-tile of 128 rows, h), h
// fastest so that CTAs running side by side touch the same 128-byte lines of
// q/k/v.  Per item it streams kv tiles of 128 residues:
//
//   warp 8  (producer)  TMA: Q tile (double buffered), then per kv tile K, V and
//                       the [128 x 128] bf16 pair-bias tile into a ring of stages
//   warp 9  (mma)       tcgen05.mma, issued in whatever order operands become
//                       ready: S = Q K^T into tensor memory and, per softmax
//                       group g, PV_g = P[:, 64g:64g+64] V[64g:64g+64, :]
//   warps 0-3, 4-7      two softmax groups.  Group g owns kv columns 64g..64g+63
//                       of every tile and runs its own online softmax over them
//                       (thread = one q row): x = S*scale*log2e + bias*log2e +
//                       mask*log2e, running max, exp2, P (bf16) to shared memory,
//                       O_g = (O_g + PV_g) * alpha.  The two partial results are
//                       merged once per item (split-kv merge) and O goes out by TMA.
//
// LSE is stored in natural log (tk_evoattention.cu:330-334).
#include "evo_host.cuh"
#include "evo_tiles.cuh"

#ifndef EVO_EXP
#define EVO_EXP 0
#endif

namespace evo {

constexpr int FWD_THREADS = 384;           // 3 warpgroups: 2 softmax + (producer, mma, 2 idle warps)
constexpr uint32_t FWD_TMEM_COLS = 256;
constexpr int FWD_REGS_SOFTMAX = 224;
constexpr int FWD_REGS_OTHER = 56;

template <int DH>
struct FwdCfg {
    static constexpr int STAGES = (DH == 32) ? 3 : 2;
    static constexpr uint32_t ROWT = RowTile<DH>::BYTES;          // one [128][DH] bf16 tile
    static constexpr uint32_t STAGE_TX = 2 * ROWT + SQ_BYTES;      // K + V + bias tile
    static constexpr uint32_t OFF_Q = 0;                           // 2 buffers
    static constexpr uint32_t OFF_K = OFF_Q + 2 * ROWT;
    static constexpr uint32_t OFF_V = OFF_K + STAGES * ROWT;
    static constexpr uint32_t OFF_BIAS = OFF_V + STAGES * ROWT;
    static constexpr uint32_t OFF_P = OFF_BIAS + STAGES * SQ_BYTES;
    static constexpr uint32_t OFF_O = OFF_P + SQ_BYTES;
    static constexpr uint32_t OFF_ML = OFF_O + ROWT;               // [2][128] float2
    static constexpr uint32_t OFF_BARS = OFF_ML + 2 * 128 * 8;
    static constexpr uint32_t NUM_BARS = 4 + 2 * STAGES + 2 + 2 + 2 + 1;
    static constexpr uint32_t OFF_MISC = OFF_BARS + NUM_BARS * 8;  // tmem slot, abort flag
    static constexpr uint32_t OFF_MASK = (OFF_MISC + 16 + 127) & ~127u;  // 2 x [NT*128] float
    static constexpr uint32_t TMEM_S = 0;
    static constexpr uint32_t TMEM_PV = 128;                       // + g * DH
};

struct FwdParams {
    int B, S, N, H;
    int QT;            // q tiles (= kv tiles) per row: ceil(N / 128)
    int total_items;   // B*S*QT*H
    float c1;          // scale * log2(e)
    const __nv_bfloat16* mask;   // [B*S][N]
    float* lse;                  // [B*S][H][N]
    __nv_bfloat16* o_resid;      // [B*S][N][H][D] or nullptr
    unsigned int* status;
};

template <int DH>
__global__ void __launch_bounds__(FWD_THREADS, 1)
evo_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_bias,
               const __grid_constant__ CUtensorMap tm_o, const FwdParams p) {
    using C = FwdCfg<DH>;
    using RT = RowTile<DH>;
    constexpr int ST = C::STAGES;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BARS);
    uint64_t* q_full = bars;                 // [2]
    uint64_t* q_empty = bars + 2;            // [2]
    uint64_t* kv_full = bars + 4;            // [ST]
    uint64_t* kv_empty = kv_full + ST;       // [ST]
    uint64_t* s_full = kv_empty + ST;        // [1]
    uint64_t* s_free = s_full + 1;           // [1]
    uint64_t* p_ready = s_free + 1;          // [2]
    uint64_t* pv_full = p_ready + 2;         // [2]
    uint64_t* grp_bar = pv_full + 2;         // [1] rendezvous of the eight softmax warps
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_MISC);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* s_mask = reinterpret_cast<float*>(smem + C::OFF_MASK);
    float2* s_ml = reinterpret_cast<float2*>(smem + C::OFF_ML);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int NT = p.QT;
    WaitCtx wc{abort_flag, p.status};

    if (tid == 0) {
        *abort_flag = 0;
        for (int i = 0; i < 2; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
        for (int i = 0; i < ST; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 9); }
        mbar_init(s_full, 1);
        mbar_init(s_free, 8);
        for (int i = 0; i < 2; ++i) { mbar_init(&p_ready[i], 4); mbar_init(&pv_full[i], 1); }
        mbar_init(grp_bar, 8);
        fence_mbar_init();
        fence_async_smem();
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot, FWD_TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == 8 && lane == 0) {
        prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v);
        prefetch_tmap(&tm_bias); prefetch_tmap(&tm_o);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    EVO_TS(t_kernel);

    const int first = blockIdx.x;
    const int stride = gridDim.x;
    const int n_items = (p.total_items > first) ? (p.total_items - first + stride - 1) / stride : 0;

    // item index -> (bs, qt, h); h fastest, then q tile, then row
    auto decode = [&](int it, int& bs, int& qt, int& h) {
        const int w = first + it * stride;
        h = w % p.H;
        const int r = w / p.H;
        qt = r % p.QT;
        bs = r / p.QT;
    };

    if (warp >= 8) {
        reg_dec<FWD_REGS_OTHER>();
        if (warp == 8 && lane == 0) {
            // ------------------------------ producer ------------------------------
            bool ok = true;
            int g = 0;   // running kv-tile counter across items
            for (int it = 0; it < n_items && ok; ++it) {
                int bs, qt, h;
                decode(it, bs, qt, h);
                const int b = bs / p.S;
                const int qb = it & 1;
                if (it >= 2) ok = mbar_wait(&q_empty[qb], ((it >> 1) - 1) & 1, wc, 0x10);
                if (!ok) break;
                mbar_arrive_expect_tx(&q_full[qb], C::ROWT);
                tma_load_4d(smem + C::OFF_Q + qb * C::ROWT, &tm_q, &q_full[qb], 0, h, qt * TILE, bs);
                for (int j = 0; j < NT; ++j, ++g) {
                    const int st = g % ST;
                    if (g >= ST) ok = mbar_wait(&kv_empty[st], ((g / ST) - 1) & 1, wc, 0x11);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&kv_full[st], C::STAGE_TX);
                    tma_load_4d(smem + C::OFF_K + st * C::ROWT, &tm_k, &kv_full[st], 0, h, j * TILE, bs);
                    tma_load_4d(smem + C::OFF_V + st * C::ROWT, &tm_v, &kv_full[st], 0, h, j * TILE, bs);
                    uint8_t* sb = smem + C::OFF_BIAS + st * SQ_BYTES;
                    tma_load_4d(sb, &tm_bias, &kv_full[st], j * TILE, qt * TILE, h, b);
                    tma_load_4d(sb + SQ_SUB_BYTES, &tm_bias, &kv_full[st], j * TILE + 64, qt * TILE, h, b);
                }
            }
            // Drain: every load issued above has landed before the CTA exits.
            const int issued = g;
            for (int k = (issued > ST ? issued - ST : 0); k < issued; ++k)
                (void)mbar_wait(&kv_full[k % ST], (k / ST) & 1, wc, 0x12);
            for (int it = (n_items > 2 ? n_items - 2 : 0); it < n_items; ++it)
                (void)mbar_wait(&q_full[it & 1], (it >> 1) & 1, wc, 0x13);
        } else if (warp == 9 && lane == 0) {
            // ------------------------------ mma issuer ------------------------------
            // Issues whichever MMA has its operands ready: S of the next tile (needs
            // its loads and the S accumulator read out) or PV_g of a tile whose P_g
            // is in shared memory.  Nothing here blocks on one barrier while
            // another piece of work could go.
            constexpr uint32_t IDESC_S = make_idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t IDESC_PV = make_idesc_bf16(128, DH, 0, 1);
            const uint32_t aQ = smem_u32(smem + C::OFF_Q), aK = smem_u32(smem + C::OFF_K);
            const uint32_t aV = smem_u32(smem + C::OFF_V), aP = smem_u32(smem + C::OFF_P);
            const int total_tiles = n_items * NT;
            int s_next = 0;
            int pv_next[2] = {0, 0};
            uint32_t idle = 0;
            uint64_t idle_t0 = 0;
            bool ok = true;
            while (ok && (pv_next[0] < total_tiles || pv_next[1] < total_tiles)) {
                bool progress = false;
                if (s_next < total_tiles) {
                    const int g = s_next;
                    const int it = g / NT, j = g - it * NT;
                    const int qb = it & 1, st = g % ST;
                    const bool rdy = (j != 0 || mbar_test(&q_full[qb], (it >> 1) & 1)) &&
                                     mbar_test(&kv_full[st], (g / ST) & 1) &&
                                     (g == 0 || mbar_test(s_free, (g - 1) & 1));
                    if (rdy) {
                        tc_fence_after();
#pragma unroll
                        for (int kb = 0; kb < RT::KBLOCKS; ++kb)
                            umma_ss(tmem + C::TMEM_S, RT::kmajor(aQ + qb * C::ROWT, kb),
                                    RT::kmajor(aK + st * C::ROWT, kb), IDESC_S, kb > 0);
                        umma_commit(s_full);
                        if (j == NT - 1) umma_commit(&q_empty[qb]);
                        ++s_next;
                        progress = true;
                    }
                }
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const int g = pv_next[w];
                    if (g < s_next && mbar_test(&p_ready[w], g & 1)) {
                        const int st = g % ST;
                        tc_fence_after();
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const int kb = 4 * w + kk;
                            umma_ss(tmem + C::TMEM_PV + w * DH, sq_kmajor(aP, kb),
                                    RT::mnmajor(aV + st * C::ROWT, kb), IDESC_PV, kk > 0);
                        }
                        umma_commit(&pv_full[w]);
                        ++pv_next[w];
                        if (pv_next[w ^ 1] > g) umma_commit(&kv_empty[st]);   // both groups' PV of tile g issued
                        progress = true;
                    }
                }
                if (progress) {
                    idle = 0;
                } else if (EVO_EXP & 16) {
                    __nanosleep(32);
                    if ((++idle & 255u) == 0u && *abort_flag) { ok = false; break; }
                } else if ((++idle & 255u) == 0u) {
                    if (*abort_flag) { ok = false; break; }
                    const uint64_t now = global_ns();
                    if (idle == 256u) idle_t0 = now;
                    if (now - idle_t0 > EVO_WAIT_NS) {
                        report(p.status, ST_WAIT_TIMEOUT, 0x2f);
                        *abort_flag = 1u;
                        ok = false;
                    }
                }
            }
        }
    } else {
        reg_inc<FWD_REGS_SOFTMAX>();
        // ------------------------------ softmax groups ------------------------------
        const int wg = warp >> 2;            // 0 or 1: kv columns 64*wg .. 64*wg+63 of each tile
        const int row = tid & 127;           // q row within the tile == TMEM lane
        const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        const int t256 = tid;                // 0..255 over both groups
        uint8_t* sP = smem + C::OFF_P;
        uint8_t* sO = smem + C::OFF_O;
        bool ok = true;
        int g = 0;
        uint32_t grp_phase = 0;
        // rendezvous of both groups (bounded)
        auto group_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(grp_bar);
            const bool r = mbar_wait(grp_bar, grp_phase, wc, 0x30);
            grp_phase ^= 1u;
            return warp_all(r);
        };

        for (int it = 0; it < n_items && ok; ++it) {
            int bs, qt, h;
            decode(it, bs, qt, h);
            float* mk = s_mask + (it & 1) * NT * TILE;
            {
                const __nv_bfloat16* src = p.mask + static_cast<size_t>(bs) * p.N;
                for (int i = t256; i < NT * TILE; i += 256)
                    mk[i] = (i < p.N) ? __bfloat162float(src[i]) * LOG2E : -INFINITY;
            }
            // The thread that issued the previous item's O store makes sure the
            // store has finished reading sO before anyone rewrites it.
            if (t256 == 0) tma_wait_group_read<0>();
            ok = group_sync();
            if (!ok) break;

            float m = -INFINITY, l = 0.f;
            float acc[DH];
#pragma unroll
            for (int i = 0; i < DH; ++i) acc[i] = 0.f;

            for (int j = 0; j < NT && ok; ++j, ++g) {
                const int st = g % ST;
                ok = warp_all(mbar_wait(s_full, g & 1, wc, 0x31));
                if (!ok) break;
                EVO_TS(t_tile);
                tc_fence_after();
                uint32_t sr[64];
                {
                    uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&sr[0]);
                    uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&sr[32]);
                    tmem_ld32(lane_base + C::TMEM_S + 64 * wg, lo);
                    tmem_ld32(lane_base + C::TMEM_S + 64 * wg + 32, hi);
                    tmem_wait_ld();
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_free);

                ok = warp_all(mbar_wait(&kv_full[st], (g / ST) & 1, wc, 0x32));
                if (!ok) break;
                const uint8_t* sb = smem + C::OFF_BIAS + st * SQ_BYTES + wg * SQ_SUB_BYTES;
                const float* mrow = mk + j * TILE + 64 * wg;
                float tmx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains: ILP
#pragma unroll
                for (int c8 = 0; c8 < 8; ++c8) {
                    const uint4 bv = *reinterpret_cast<const uint4*>(sb + swz_off<128>(row, c8));
                    const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                    for (int q4 = 0; q4 < 2; ++q4) {
                        const float4 mv = *reinterpret_cast<const float4*>(mrow + c8 * 8 + q4 * 4);
                        const float mm[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = c8 * 8 + q4 * 4 + e;
                            const uint32_t word = bw[q4 * 2 + (e >> 1)];
                            const float bval = (e & 1) ? bf16_hi(word) : bf16_lo(word);
                            const float x = fmaf(__uint_as_float(sr[c]), p.c1, fmaf(bval, LOG2E, mm[e]));
                            sr[c] = __float_as_uint(x);
                            tmx[e] = fmaxf(tmx[e], x);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&kv_empty[st]);

                const float tmax = fmaxf(fmaxf(tmx[0], tmx[1]), fmaxf(tmx[2], tmx[3]));
                const float m_new = fmaxf(m, tmax);
                const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
                const float alpha = ex2(m - m_safe);
                float rs[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const float pv = ex2(__uint_as_float(sr[c]) - m_safe);
                    rs[c & 3] += pv;
                    sr[c] = __float_as_uint(pv);
                }
                l = l * alpha + ((rs[0] + rs[1]) + (rs[2] + rs[3]));
                m = m_new;

                if (j > 0) {
                    // PV of the previous tile: also tells us its MMA no longer reads sP.
                    ok = warp_all(mbar_wait(&pv_full[wg], (g - 1) & 1, wc, 0x33));
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < DH / 32; ++c) {
                        uint32_t r[32];
                        tmem_ld32(lane_base + C::TMEM_PV + wg * DH + c * 32, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            acc[c * 32 + i] = (acc[c * 32 + i] + __uint_as_float(r[i])) * alpha;
                    }
                }
                // P (bf16) into this group's [128][64] sub-tile of the square tile.
#pragma unroll
                for (int c8 = 0; c8 < 8; ++c8) {
                    uint4 v;
                    v.x = pack_bf16(__uint_as_float(sr[c8 * 8 + 0]), __uint_as_float(sr[c8 * 8 + 1]));
                    v.y = pack_bf16(__uint_as_float(sr[c8 * 8 + 2]), __uint_as_float(sr[c8 * 8 + 3]));
                    v.z = pack_bf16(__uint_as_float(sr[c8 * 8 + 4]), __uint_as_float(sr[c8 * 8 + 5]));
                    v.w = pack_bf16(__uint_as_float(sr[c8 * 8 + 6]), __uint_as_float(sr[c8 * 8 + 7]));
                    *reinterpret_cast<uint4*>(sP + wg * SQ_SUB_BYTES + swz_off<128>(row, c8)) = v;
                }
                fence_async_smem();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_ready[wg]);
                EVO_TE(t_tile, p.status, 0x78);
            }
            if (!ok) break;
            EVO_TS(t_epi);
            // last tile's PV
            ok = warp_all(mbar_wait(&pv_full[wg], (g - 1) & 1, wc, 0x34));
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < DH / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(lane_base + C::TMEM_PV + wg * DH + c * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[c * 32 + i] += __uint_as_float(r[i]);
            }
            tc_fence_before();

            // ---- merge the two groups' partial softmax results ----
            // Group g finalises output columns [g*DH/2, (g+1)*DH/2): it hands the
            // other half of its accumulator to the other group through its own
            // (now idle) half of the P tile.
            constexpr int HALF = DH / 2;                  // floats per row handed over
            constexpr int XCH = HALF / 4;                 // 16-byte chunks per row
            const int other = wg ^ 1;
            // keep[] = the half this group finalises, give[] = the half it hands over
            float keep[HALF], give[HALF];
#pragma unroll
            for (int i = 0; i < HALF; ++i) {
                keep[i] = wg ? acc[HALF + i] : acc[i];
                give[i] = wg ? acc[i] : acc[HALF + i];
            }
            {
                uint8_t* mine = sP + wg * SQ_SUB_BYTES;
#pragma unroll
                for (int c = 0; c < XCH; ++c) {
                    float4 v = make_float4(give[c * 4 + 0], give[c * 4 + 1], give[c * 4 + 2], give[c * 4 + 3]);
                    *reinterpret_cast<float4*>(mine + swz_off<HALF * 4>(row, c)) = v;
                }
                s_ml[wg * 128 + row] = make_float2(m, l);
            }
            ok = group_sync();
            if (!ok) break;
            {
                const float2 ml_o = s_ml[other * 128 + row];
                const float mt = fmaxf(m, ml_o.x);      // finite: column 0 of tile 0 is never -inf
                const float f = ex2(m - mt), fo = ex2(ml_o.x - mt);
                const float lt = l * f + ml_o.y * fo;
                const float inv = 1.f / lt;
                const uint8_t* theirs = sP + other * SQ_SUB_BYTES;
                float outv[HALF];
#pragma unroll
                for (int c = 0; c < XCH; ++c) {
                    const float4 v = *reinterpret_cast<const float4*>(theirs + swz_off<HALF * 4>(row, c));
                    outv[c * 4 + 0] = (keep[c * 4 + 0] * f + v.x * fo) * inv;
                    outv[c * 4 + 1] = (keep[c * 4 + 1] * f + v.y * fo) * inv;
                    outv[c * 4 + 2] = (keep[c * 4 + 2] * f + v.z * fo) * inv;
                    outv[c * 4 + 3] = (keep[c * 4 + 3] * f + v.w * fo) * inv;
                }
                const int qrow = qt * TILE + row;
                // bf16 row into the O staging tile (same swizzle as a row tile); the
                // rounding residual goes straight to global memory
#pragma unroll
                for (int c8 = 0; c8 < HALF / 8; ++c8) {
                    uint4 v;
                    v.x = pack_bf16(outv[c8 * 8 + 0], outv[c8 * 8 + 1]);
                    v.y = pack_bf16(outv[c8 * 8 + 2], outv[c8 * 8 + 3]);
                    v.z = pack_bf16(outv[c8 * 8 + 4], outv[c8 * 8 + 5]);
                    v.w = pack_bf16(outv[c8 * 8 + 6], outv[c8 * 8 + 7]);
                    const int chunk = wg * (HALF / 8) + c8;   // 16-byte chunk within the row
                    *reinterpret_cast<uint4*>(sO + swz_off<RT::ROW_BYTES>(row, chunk)) = v;
                    if (p.o_resid != nullptr && qrow < p.N) {
                        const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
                        uint32_t rw[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            rw[e] = pack_bf16(outv[c8 * 8 + 2 * e] - bf16_lo(vw[e]),
                                              outv[c8 * 8 + 2 * e + 1] - bf16_hi(vw[e]));
                        __nv_bfloat16* dst = p.o_resid +
                            ((static_cast<size_t>(bs) * p.N + qrow) * p.H + h) * DH + wg * HALF + c8 * 8;
                        *reinterpret_cast<uint4*>(dst) = make_uint4(rw[0], rw[1], rw[2], rw[3]);
                    }
                }
                if (wg == 0 && qrow < p.N)
                    p.lse[(static_cast<size_t>(bs) * p.H + h) * p.N + qrow] = mt * LN2 + __logf(lt);
            }
            fence_async_smem();
            ok = group_sync();
            if (!ok) break;
            if (t256 == 0) {
                tma_store_4d(&tm_o, sO, 0, h, qt * TILE, bs);
                tma_commit_group();
            }
            EVO_TE(t_epi, p.status, 0x79);
        }
        if (t256 == 0) tma_wait_group<0>();
    }

    if (tid == 0) EVO_TE(t_kernel, p.status, 0x7e);
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem, FWD_TMEM_COLS);
}

template <int DH>
static int launch_fwd(const EvoDims* d, const void* q, const void* k, const void* v, const void* bias,
                      const void* mask, void* o, void* o_resid, float* lse, float scale, cudaStream_t st) {
    using C = FwdCfg<DH>;
    const int BS = d->B * d->S;
    const int QT = (d->N + TILE - 1) / TILE;
    const size_t smem = 1024 + C::OFF_MASK + static_cast<size_t>(2) * QT * TILE * sizeof(float);
    if (smem > 232448) return EVO_ERR_BAD_DIMS;

    CUtensorMap tq, tk, tv, tb, to;
    int rc;
    if ((rc = make_tmap_qkv(&tq, q, BS, d->N, d->H, DH, TILE))) return rc;
    if ((rc = make_tmap_qkv(&tk, k, BS, d->N, d->H, DH, TILE))) return rc;
    if ((rc = make_tmap_qkv(&tv, v, BS, d->N, d->H, DH, TILE))) return rc;
    if ((rc = make_tmap_bias(&tb, bias, d->B, d->H, d->N))) return rc;
    if ((rc = make_tmap_qkv(&to, o, BS, d->N, d->H, DH, TILE))) return rc;

    FwdParams p;
    p.B = d->B; p.S = d->S; p.N = d->N; p.H = d->H;
    p.QT = QT;
    p.total_items = BS * QT * d->H;
    p.c1 = ((scale > 0.f) ? scale : 1.0f / sqrtf(static_cast<float>(DH))) * LOG2E;
    p.mask = static_cast<const __nv_bfloat16*>(mask);
    p.lse = lse;
    p.o_resid = static_cast<__nv_bfloat16*>(o_resid);
    p.status = status_word();
    if (!p.status) return EVO_ERR_CUDA;

    int dev = 0, sms = 0;
    if ((rc = cuda_err(cudaGetDevice(&dev)))) return rc;
    if ((rc = cuda_err(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)))) return rc;
    if ((rc = cuda_err(cudaFuncSetAttribute(evo_fwd_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(smem)))))
        return rc;
    const int grid = p.total_items < sms ? p.total_items : sms;
    prof_begin(0, st);
    evo_fwd_kernel<DH><<<grid, FWD_THREADS, smem, st>>>(tq, tk, tv, tb, to, p);
    prof_end(0, st);
    return cuda_err(cudaGetLastError());
}

}  // namespace evo

extern "C" int evo_fwd(const EvoDims* dims, const void* q, const void* k, const void* v,
                       const void* pair_bias, const void* res_mask, void* o, void* o_resid, float* lse,
                       float scale, void* stream) {
    int rc = evo::check_dims(dims);
    if (rc) return rc;
    if (!q || !k || !v || !pair_bias || !res_mask || !o || !lse) return EVO_ERR_NULL_PTR;
    const uintptr_t all = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                          reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(pair_bias) |
                          reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(o_resid);
    if (all & 15u) return EVO_ERR_ALIGNMENT;
    if ((rc = evo::ensure_context())) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dims->D == 32)
        return evo::launch_fwd<32>(dims, q, k, v, pair_bias, res_mask, o, o_resid, lse, scale, st);
    return evo::launch_fwd<64>(dims, q, k, v, pair_bias, res_mask, o, o_resid, lse, scale, st);
}
