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
// q/k/v.  Per item it streams kv tiles of 128 residues (NG = 2 softmax groups):
//
//   warp 8  (producer)  TMA: Q tile (double buffered; one buffer at D = 128), then per
//                       kv tile K, V, the [128 x 128] bf16 pair-bias tile (D <= 64)
//                       and the mask row into a ring of stages
//   warp 9  (S issuer)  tcgen05.mma S_g = Q K[64g:64g+64, :]^T into tensor memory for
//                       each softmax group g, a tile ahead of the softmax (two buffers)
//   warp 10 (PV issuer) PV_g (+)= P_g V[64g:64g+64, :] with P_g read from tensor
//                       memory; the accumulator stays in tensor memory for the item.
//                       The groups share no barrier inside an item, so they drift
//                       apart and one group's exp2 phase overlaps the other's FMA phase
//   warps 0-3, 4-7      two softmax groups.  Group g owns kv columns 64g..64g+63
//                       of every tile and runs its own online softmax over them
//                       (thread = one q row): x = S*scale*log2e + bias*log2e +
//                       mask*log2e, running max, exp2, P (bf16) back into tensor
//                       memory; when the row maximum rises the accumulator is
//                       rescaled in place.  After an item each group publishes its
//                       (m, l); each group then merges, normalises and stores half of
//                       the head-dim columns of O, reading both groups' accumulators.
//                       That epilogue is deferred into the next item's first tile, so
//                       the last PV of an item is never waited for idly.
//
// LSE is stored in natural log (tk_evoattention.cu:330-334).
#include "evo_host.cuh"
#include "evo_tiles.cuh"

namespace evo {

// How far the running row maximum may fall behind before the accumulator in tensor memory is
// rescaled.  0 = the exact online softmax: the largest P of a row is exp2(0) = 1, which bf16
// represents exactly, so a row dominated by one logit carries no rounding error from its main
// term.  A lag of 8 (P up to 256, the rescale then almost never runs) measured 2 % faster but
// put a 2^-9 relative error on exactly those main terms: 10x the dBias error at heavy-tailed
// logits (0.033 against 0.0035 max-abs at B=1, S=48, N=768, H=8, D=32, bias std 2).
#ifndef EVO_FWD_LAZY
#define EVO_FWD_LAZY 0.0f
#endif
// Softmax groups per CTA.  A group is four warps (thread = one q row) that own kv columns
// g*CW .. g*CW+CW-1 (CW = 128 / NG) of every tile and run their own online softmax over them; the
// groups' partial results are merged in the epilogue.  NG = 2 is the general form.  NG = 4 (D = 32
// only: tensor memory holds four accumulators of 32 columns, not of 64) puts four softmax warps on
// every scheduler, so that two of them can keep the exp2 unit saturated while the other two are in
// the fused-multiply-add pass of their tile.
template <int DH, int NG>
struct FwdCfg {
    static_assert(NG == 2 || NG == 4, "two or four softmax groups");
    static constexpr int CW = TILE / NG;                       // kv columns per group
    static constexpr int NSW = NG * 4;                         // softmax warps
    // + an epilogue warpgroup (warps NSW .. NSW+3: warp & 3 is its quarter of the tensor-memory
    // lanes) + a warpgroup of producer, S issuer, PV issuer and one idle warp
    static constexpr int THREADS = (NSW + 8) * 32;
    // setmaxnreg budgets (one value per warpgroup): the CTA's register pool is the launch count (the
    // cap ptxas derives from the launch bound) times the threads; an increase that the pool cannot
    // satisfy blocks for ever
    static constexpr int REGS_LAUNCH = (65536 / THREADS) & ~7;
    // Measured at B=1, S=512, N=384, H=8, D=32 (forward kernel): 208/40/40 0.392 ms, 200/56/56 0.393,
    // 200/72/40 0.383, 192/72/56 0.376, 192/64/64 0.370, 184/72/72 0.383, 176/80/80 0.378.
#ifndef EVO_FWD_RS
#define EVO_FWD_RS 192
#define EVO_FWD_RE 64
#define EVO_FWD_RO 64
#endif
    static constexpr int REGS_SOFTMAX = (NG == 2) ? EVO_FWD_RS : 96;
    static constexpr int REGS_EPI = (NG == 2) ? EVO_FWD_RE : 40;
    static constexpr int REGS_OTHER = (NG == 2) ? EVO_FWD_RO : 40;
    static_assert((REGS_SOFTMAX * NSW + REGS_EPI * 4 + REGS_OTHER * 4) * 32 <= REGS_LAUNCH * THREADS, "register pool");
    static constexpr int STAGES = (DH == 32) ? 3 : 2;
    static constexpr uint32_t ROWT = RowTile<DH>::BYTES;          // one [128][DH] bf16 tile
    // D = 128 is short of shared and tensor memory: one Q buffer instead of two, the bias slice of
    // a thread read straight from global memory instead of a staged tile, and P (bf16) written
    // over the S columns it was computed from (S of tile j+2 then waits for PV of tile j).
    static constexpr bool WIDE = (DH == 128);
    static constexpr int NQ = WIDE ? 1 : 2;                        // Q buffers
    static constexpr uint32_t BIAS_BYTES = WIDE ? 0 : SQ_BYTES;
    // one stage: K tile, V tile, bias tile (two [128][64] halves), raw bf16 mask row
    static constexpr uint32_t ST_K = 0, ST_V = ROWT, ST_BIAS = 2 * ROWT, ST_MASK = 2 * ROWT + BIAS_BYTES;
    static constexpr uint32_t STAGE_STRIDE = 2 * ROWT + BIAS_BYTES + 1024;
    static constexpr uint32_t OFF_Q = 0;                           // NQ buffers
    static constexpr uint32_t OFF_STAGE = OFF_Q + NQ * ROWT;
    // O staging: one row tile, written by the epilogue warpgroup, sent out by TMA
    static constexpr uint32_t OFF_O = OFF_STAGE + STAGES * STAGE_STRIDE;
    // exchange of the groups' (m, l) per row: [item parity][group][128 rows]
    static constexpr uint32_t OFF_XCH = OFF_O + ROWT;
    static constexpr uint32_t OFF_WMASK = OFF_XCH + 2 * NG * 128 * 8;      // NSW warps x CW floats
    static constexpr uint32_t OFF_BARS = OFF_WMASK + NSW * CW * 4;
    static constexpr uint32_t NUM_BARS = 4 + 2 * STAGES + 4 * NG + 2 * NG + 2 * NG + 3 + 2;
    static constexpr uint32_t OFF_MISC = OFF_BARS + NUM_BARS * 8;
    static constexpr uint32_t SMEM_BYTES = OFF_MISC + 16 + 1024;   // + alignment slack
    static constexpr uint32_t TMEM_S = 0;                          // two buffers: + (tile & 1) * 128 + g * CW
    static constexpr uint32_t TMEM_PV = 256;                       // + g * DH
    static constexpr uint32_t TMEM_P = 256 + NG * DH;              // + g * CW/2: CW bf16 per lane (not WIDE)
    static constexpr uint32_t TMEM_COLS = 512;
    static_assert(WIDE ? (TMEM_PV + NG * DH <= TMEM_COLS) : (TMEM_P + 64 <= TMEM_COLS), "tensor memory budget");
    // tensor-memory column (without the lane part) of group w's P of running tile g
    __device__ static __forceinline__ uint32_t p_col(int w, int g) {
        return WIDE ? TMEM_S + (g & 1) * 128 + CW * w : TMEM_P + w * (CW / 2);
    }
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
    static_assert(OFF_STAGE % 1024 == 0 && STAGE_STRIDE % 1024 == 0 && OFF_O % 1024 == 0, "tile alignment");
};

struct FwdParams {
    int B, S, N, H;
    int Dt;            // true head dim (16 runs on the D = 32 kernel: loads zero-filled, stores clipped)
    int KB;            // contraction blocks of 16 head-dim columns that hold data: ceil(Dt / 16)
    int QT;            // q tiles (= kv tiles) per row: ceil(N / 128)
    int total_items;   // B*S*QT*H
    float c1;          // scale * log2(e)
    const __nv_bfloat16* mask;   // [B*S][N]
    const __nv_bfloat16* bias;   // [B][H][N][N] (read directly when the bias tile is not staged)
    float* lse;                  // [B*S][H][N]
    __nv_bfloat16* o_resid;      // activation layout `lay`, or nullptr
    const __nv_bfloat16* gate;   // activation layout `lay`, or nullptr: pre-activation gate logits
    __nv_bfloat16* o_gated;      // activation layout `lay` (with gate): O * sigmoid(gate)
    ActLayout lay;               // element strides of the activation tensors
    unsigned int* status;
};

// STRIDED: the activation tensors are views with the strides of p.lay; otherwise they are
// contiguous and the residual's address is formed from N and H alone.  (The generic address
// arithmetic, in the epilogue, cost 4-10 % of the kernel when it was the only version: the
// contiguous case keeps its own instantiation.)
// GATED: the epilogue also writes sigmoid(gate) * O (its own instantiation: the extra loads and
// arithmetic, even behind a uniform branch, cost the plain kernel 5 %).
template <int DH, bool STRIDED, int NG, bool GATED>
__global__ void __launch_bounds__((FwdCfg<DH, NG>::THREADS), 1)
evo_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_bias,
               const __grid_constant__ CUtensorMap tm_o, const FwdParams p) {
    using C = FwdCfg<DH, NG>;
    using RT = RowTile<DH>;
    constexpr int ST = C::STAGES, CW = C::CW, NSW = C::NSW;
    constexpr int W_EPI = NSW, W_PROD = NSW + 4, W_S = NSW + 5, W_PV = NSW + 6;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BARS);
    uint64_t* q_full = bars;                 // [2]
    uint64_t* q_empty = bars + 2;            // [2]
    uint64_t* kv_full = bars + 4;            // [ST]
    uint64_t* kv_empty = kv_full + ST;       // [ST]
    uint64_t* s_full = kv_empty + ST;        // [2 * NG]: softmax group + NG * S buffer
    uint64_t* s_free = s_full + 2 * NG;      // [2 * NG]
    uint64_t* p_ready = s_free + 2 * NG;     // [NG] per softmax group
    uint64_t* pv_full = p_ready + NG;        // [NG]
    uint64_t* xch_ready = pv_full + NG;      // [item parity][group]: the group's final (m, l) of an item are written
    uint64_t* acc_full = xch_ready + 2 * NG; // every PV MMA of an item is complete
    uint64_t* acc_free = acc_full + 1;       // the epilogue has read the item's accumulators and (m, l)
    uint64_t* e_bar = acc_free + 1;          // rendezvous of the four epilogue warps
    uint64_t* xu_done = e_bar + 1;           // [2]: a half of the groups has finished the exp2 pass of a tile
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_MISC);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int NT = p.QT;
    WaitCtx wc{abort_flag, p.status};

    if (tid == 0) {
        *abort_flag = 0;
        for (int i = 0; i < 2; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
        for (int i = 0; i < ST; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], NSW + 1); }
        for (int i = 0; i < 2 * NG; ++i) {
            mbar_init(&s_full[i], 1); mbar_init(&s_free[i], C::WIDE ? 1 : 4); mbar_init(&xch_ready[i], 4);
        }
        for (int i = 0; i < NG; ++i) { mbar_init(&p_ready[i], 4); mbar_init(&pv_full[i], 1); }
        mbar_init(acc_full, 1);
        mbar_init(acc_free, 4);
        mbar_init(e_bar, 4);
        for (int i = 0; i < 2; ++i) mbar_init(&xu_done[i], NSW / 2);
        fence_mbar_init();
        fence_async_smem();
    }
    if (warp == W_S) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == W_PROD && lane == 0) {
        prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v);
        prefetch_tmap(&tm_bias); prefetch_tmap(&tm_o);
    }
    EVO_TRACE_INIT();
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

    if (warp >= NSW + 4) {
        reg_dec<C::REGS_OTHER>();
        if (warp == W_PROD) {
            if (lane == 0) {
                // ------------------------------ producer ------------------------------
                bool ok = true;
                int g = 0;   // running kv-tile counter across items
                for (int it = 0; it < n_items && ok; ++it) {
                    int bs, qt, h;
                    decode(it, bs, qt, h);
                    const int b = bs / p.S;
                    const int qb = it % C::NQ;
                    if (it >= C::NQ) ok = mbar_wait(&q_empty[qb], ((it / C::NQ) - 1) & 1, wc, 0x10);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&q_full[qb], C::ROWT);
                    tma_load_row_tile<DH>(smem + C::OFF_Q + qb * C::ROWT, &tm_q, &q_full[qb], h, qt * TILE, bs);
                    for (int j = 0; j < NT; ++j, ++g) {
                        const int st = g % ST;
                        if (g >= ST) ok = mbar_wait(&kv_empty[st], ((g / ST) - 1) & 1, wc, 0x11);
                        if (!ok) break;
                        uint8_t* sb = smem + C::OFF_STAGE + st * C::STAGE_STRIDE;
                        const int ncol = (p.N - j * TILE < TILE) ? (p.N - j * TILE) : TILE;   // multiple of 8
                        mbar_arrive_expect_tx(&kv_full[st], 2 * C::ROWT + C::BIAS_BYTES + ncol * 2);
                        tma_load_row_tile<DH>(sb + C::ST_K, &tm_k, &kv_full[st], h, j * TILE, bs);
                        tma_load_row_tile<DH>(sb + C::ST_V, &tm_v, &kv_full[st], h, j * TILE, bs);
                        if (!C::WIDE) {
                            tma_load_4d(sb + C::ST_BIAS, &tm_bias, &kv_full[st], j * TILE, qt * TILE, h, b);
                            tma_load_4d(sb + C::ST_BIAS + SQ_SUB_BYTES, &tm_bias, &kv_full[st], j * TILE + 64, qt * TILE, h, b);
                        }
                        bulk_load(sb + C::ST_MASK, p.mask + static_cast<size_t>(bs) * p.N + j * TILE, ncol * 2, &kv_full[st]);
                    }
                }
                // Drain: every load issued above has landed before the CTA exits.
                const int issued = g;
                for (int k = (issued > ST ? issued - ST : 0); k < issued; ++k)
                    (void)mbar_wait(&kv_full[k % ST], (k / ST) & 1, wc, 0x12);
                for (int it = (n_items > C::NQ ? n_items - C::NQ : 0); it < n_items; ++it)
                    (void)mbar_wait(&q_full[it % C::NQ], (it / C::NQ) & 1, wc, 0x13);
            }
        } else if (warp == W_S) {
            // ------------------------------ S issuer ------------------------------
            // S_w = Q K[CW w : CW w + CW, :]^T for every softmax group w of every tile, one tile ahead
            // of the softmax (two S buffers).  The warp runs its loop with all lanes (uniform control
            // flow keeps the operand descriptors in uniform registers) and elects one lane to issue.
            constexpr uint32_t IDESC_S = make_idesc_bf16(128, CW, 0, 0);
            const uint32_t aQ = smem_u32(smem + C::OFF_Q), aSt = smem_u32(smem + C::OFF_STAGE);
            bool ok = true;
            int g = 0;
            for (int it = 0; it < n_items && ok; ++it) {
                const int qb = it % C::NQ;
                for (int j = 0; j < NT && ok; ++j, ++g) {
                    const int st = g % ST;
                    if (j == 0) ok = warp_all(mbar_wait(&q_full[qb], (it / C::NQ) & 1, wc, 0x20));
                    if (ok) ok = warp_all(mbar_wait(&kv_full[st], (g / ST) & 1, wc, 0x21));
#pragma unroll
                    for (int w = 0; w < NG; ++w) {
                        const int sb = w + NG * (g & 1);
                        if (ok && g >= 2) ok = warp_all(mbar_wait(&s_free[sb], ((g >> 1) - 1) & 1, wc, 0x22));
                        if (!ok) break;
                        tc_fence_after();
                        if (elect_one()) {
                            // K rows CW w .. of the tile: that many rows further into the K-major tile
                            const uint32_t kt = aSt + st * C::STAGE_STRIDE + C::ST_K + w * CW * RT::ROW_BYTES;
#pragma unroll
                            for (int kb = 0; kb < RT::KBLOCKS; ++kb)
                                if (kb < p.KB)      // blocks past the true head dim are zero-filled: skipped
                                    umma_ss(tmem + C::TMEM_S + (g & 1) * 128 + CW * w, RT::kmajor(aQ + qb * C::ROWT, kb),
                                            RT::kmajor(kt, kb), IDESC_S, kb > 0);
                            umma_commit(&s_full[sb]);
                            // Q is free once every group's S of the item's last tile is issued
                            if (w == NG - 1 && j == NT - 1) umma_commit(&q_empty[qb]);
                        }
                        __syncwarp();
                    }
                }
            }
        } else if (warp == W_PV) {
            // ------------------------------ PV issuer ------------------------------
            // PV_w (+)= P_w V[CW w : CW w + CW, :] with P_w read from tensor memory; the accumulator of a
            // group stays in tensor memory for the whole item (the first tile overwrites it).
            const uint32_t IDESC_PV = make_idesc_bf16(128, 16 * p.KB, 0, 1);   // N = the head-dim columns that hold data
            const uint32_t aSt = smem_u32(smem + C::OFF_STAGE);
            bool ok = true;
            int g = 0;
            for (int it = 0; it < n_items && ok; ++it) {
                for (int j = 0; j < NT && ok; ++j, ++g) {
                    const int st = g % ST;
                    // the first PV of an item overwrites the accumulators: the epilogue has read the previous item's
                    if (j == 0 && it > 0) ok = warp_all(mbar_wait(acc_free, (it - 1) & 1, wc, 0x24));
#pragma unroll
                    for (int w = 0; w < NG; ++w) {
                        if (ok) ok = warp_all(mbar_wait(&p_ready[w], g & 1, wc, 0x23));
                        if (!ok) break;
                        tc_fence_after();
                        if (elect_one()) {
#pragma unroll
                            for (int kk = 0; kk < CW / 16; ++kk)
                                umma_ts(tmem + C::TMEM_PV + w * DH, tmem + C::p_col(w, g) + kk * 8,
                                        RT::mnmajor(aSt + st * C::STAGE_STRIDE + C::ST_V, (CW / 16) * w + kk), IDESC_PV,
                                        (kk > 0 || j > 0) ? 1u : 0u);
                            umma_commit(&pv_full[w]);
                            if (C::WIDE) umma_commit(&s_free[w + NG * (g & 1)]);   // P sat in this S buffer
                            if (w == NG - 1) umma_commit(&kv_empty[st]);   // every group's PV of the tile issued
                            if (w == NG - 1 && j == NT - 1) umma_commit(acc_full);   // ... and of the item
                        }
                        __syncwarp();
                    }
                }
            }
        }
    } else if (warp >= W_EPI) {
        reg_dec<C::REGS_EPI>();
        // ------------------------------ epilogue warpgroup ------------------------------
        // Finishes item k while the softmax groups are already in item k+1: merges the groups'
        // partial results (split-kv merge), normalises, writes O through shared memory and TMA, the
        // log-sum-exp, the rounding residual and the gated output.  Thread = one q row; warp e reads
        // tensor-memory lanes 32e .. 32e+31.
        const int row = tid & 127;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        const uint32_t aO = smem_u32(smem + C::OFF_O);
        const uint32_t aXch = smem_u32(smem + C::OFF_XCH);
        bool ok = true;
        uint32_t e_phase = 0;
        auto epi_sync = [&]() -> bool {      // rendezvous of the four epilogue warps (bounded)
            __syncwarp();
            if (lane == 0) mbar_arrive(e_bar);
            const bool r = warp_all(mbar_wait(e_bar, e_phase, wc, 0x30));
            e_phase ^= 1u;
            return r;
        };
        constexpr int EC = 16;               // head-dim columns per pass (register budget)
        for (int it = 0; it < n_items && ok; ++it) {
            int bs, qt, h;
            decode(it, bs, qt, h);
            EVO_TS(t_epi);
            const int qrow = qt * TILE + row;
            size_t act_off;
            if constexpr (STRIDED)
                act_off = bs * p.lay.row + qrow * p.lay.n + h * p.lay.h;
            else
                act_off = ((static_cast<size_t>(bs) * p.N + qrow) * p.H + h) * DH;
            // every group's (m, l) of the item, then every PV MMA of the item
            float gm[NG], gl[NG];
#pragma unroll
            for (int og = 0; og < NG; ++og) {
                if (ok) ok = warp_all(mbar_wait(&xch_ready[(it & 1) * NG + og], (it >> 1) & 1, wc, 0x35));
                if (!ok) break;
                asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(gm[og]), "=f"(gl[og])
                             : "r"(aXch + (((it & 1) * NG + og) * 128 + row) * 8));
            }
            if (ok) ok = warp_all(mbar_wait(acc_full, it & 1, wc, 0x37));
            if (!ok) break;
            tc_fence_after();
            float mt = gm[0];
#pragma unroll
            for (int og = 1; og < NG; ++og) mt = fmaxf(mt, gm[og]);
            const float ms = (mt == -INFINITY) ? 0.f : mt;
            float gf[NG], lt = 0.f;
#pragma unroll
            for (int og = 0; og < NG; ++og) { gf[og] = ex2(gm[og] - ms); lt += gl[og] * gf[og]; }
            const float inv = 1.f / lt;
#pragma unroll
            for (int og = 0; og < NG; ++og) gf[og] *= inv;
            // the previous item's TMA store must have finished reading the staging tile
            if (row == 0) tma_wait_group_read<0>();
            if (!epi_sync()) { ok = false; break; }
#pragma unroll
            for (int hc = 0; hc < DH / EC; ++hc) {
                float outv[EC];
#pragma unroll
                for (int e = 0; e < EC; ++e) outv[e] = 0.f;
#pragma unroll
                for (int og = 0; og < NG; ++og) {
                    float part[EC];
                    tmem_ld_f32<EC>(lane_base + C::TMEM_PV + og * DH + hc * EC, part);
#pragma unroll
                    for (int e = 0; e < EC; ++e) outv[e] = fmaf(part[e], gf[og], outv[e]);
                }
                if (hc == DH / EC - 1) {
                    // accumulators and (m, l) are read: the next item's first PV may overwrite them
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_free);
                }
#pragma unroll
                for (int c8l = 0; c8l < EC / 8; ++c8l) {
                    const int col = hc * EC + c8l * 8;                 // first head-dim column of this 16-byte chunk
                    uint4 v;
                    v.x = pack_bf16(outv[c8l * 8 + 0], outv[c8l * 8 + 1]);
                    v.y = pack_bf16(outv[c8l * 8 + 2], outv[c8l * 8 + 3]);
                    v.z = pack_bf16(outv[c8l * 8 + 4], outv[c8l * 8 + 5]);
                    v.w = pack_bf16(outv[c8l * 8 + 6], outv[c8l * 8 + 7]);
                    sts128(aO + (col / RT::BOX_D) * RT::SUB_BYTES + swz_off<RT::ROW_BYTES>(row, (col % RT::BOX_D) / 8), v);
                    if (qrow < p.N && col < p.Dt) {
                        if (p.o_resid != nullptr) {
                            // rounding residual of O, straight to global memory
                            const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
                            uint32_t rw[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                rw[e] = pack_bf16(outv[c8l * 8 + 2 * e] - bf16_lo(vw[e]),
                                                  outv[c8l * 8 + 2 * e + 1] - bf16_hi(vw[e]));
                            *reinterpret_cast<uint4*>(p.o_resid + act_off + col) = make_uint4(rw[0], rw[1], rw[2], rw[3]);
                        }
                        if constexpr (GATED) {
                            // O * sigmoid(gate), from the unrounded O
                            const uint4 g4 = __ldg(reinterpret_cast<const uint4*>(p.gate + act_off + col));
                            const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w};
                            uint32_t ow[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float s0 = 1.0f / (1.0f + ex2(-bf16_lo(gw[e]) * LOG2E));
                                const float s1 = 1.0f / (1.0f + ex2(-bf16_hi(gw[e]) * LOG2E));
                                ow[e] = pack_bf16(outv[c8l * 8 + 2 * e] * s0, outv[c8l * 8 + 2 * e + 1] * s1);
                            }
                            *reinterpret_cast<uint4*>(p.o_gated + act_off + col) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                        }
                    }
                }
            }
            if (qrow < p.N) p.lse[(static_cast<size_t>(bs) * p.H + h) * p.N + qrow] = ms * LN2 + __logf(lt);
            fence_async_smem();
            if (!epi_sync()) { ok = false; break; }
            if (row == 0) {
#pragma unroll
                for (int sub = 0; sub < RT::SUBS; ++sub)
                    if (sub * RT::BOX_D < p.Dt)
                        tma_store_4d(&tm_o, smem + C::OFF_O + sub * RT::SUB_BYTES, sub * RT::BOX_D, h, qt * TILE, bs);
                tma_commit_group();
            }
            EVO_TE(t_epi, p.status, 0x79);
        }
        if (row == 0) tma_wait_group<0>();
    } else {
        reg_inc<C::REGS_SOFTMAX>();
        // ------------------------------ softmax groups ------------------------------
        const int wg = warp >> 2;            // kv columns CW*wg .. CW*wg+CW-1 of each tile
        const int row = tid & 127;           // q row within the tile == TMEM lane
        const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        const uint32_t aStage = smem_u32(smem + C::OFF_STAGE);
        const uint32_t aXch = smem_u32(smem + C::OFF_XCH);            // [parity][group][128 rows] (m, l)
        const uint32_t aWmask = smem_u32(smem + C::OFF_WMASK) + warp * CW * 4;
        const uint32_t scratch_w = smem_u32(tmem_slot + 2);           // a word nobody reads
        const float2 c1x2 = make_float2(p.c1, p.c1), l2e2 = make_float2(LOG2E, LOG2E);
        // where this group's columns sit in the bias tile (two [128][64] sub-tiles, 16-byte chunks)
        constexpr int CH0_MASK = 7;
        const uint32_t bias_sub = ((CW * wg) >> 6) * SQ_SUB_BYTES;
        const int bias_c0 = ((CW * wg) & 63) >> 3;
        (void)CH0_MASK;
        bool ok = true;
        int g = 0;
        float m_used = -INFINITY, l = 0.f;

        for (int it = 0; it < n_items && ok; ++it) {
            int bs, qt, h;
            decode(it, bs, qt, h);
            m_used = -INFINITY;
            l = 0.f;
            for (int j = 0; j < NT && ok; ++j, ++g) {
                const int st = g % ST;
                const uint32_t sb = aStage + st * C::STAGE_STRIDE;
                const int sbuf = wg + NG * (g & 1);
                const uint32_t tS = lane_base + C::TMEM_S + (g & 1) * 128 + CW * wg;
                if ((warp & 3) == 0 && wg < 3) EVO_TL(p.status, 5 + wg, g, 0);
                // without a staged bias tile: this thread's CW bias values of the tile, straight from
                // global memory, requested before the wait so that they arrive while the MMA runs
                uint4 bg[C::WIDE ? CW / 8 : 1];
                if constexpr (C::WIDE) {
                    const int qrow = qt * TILE + row, col0 = j * TILE + CW * wg;
                    const __nv_bfloat16* bp =
                        p.bias + ((static_cast<size_t>(bs / p.S) * p.H + h) * p.N + qrow) * p.N + col0;
#pragma unroll
                    for (int c8 = 0; c8 < CW / 8; ++c8) {
                        bg[c8] = make_uint4(0u, 0u, 0u, 0u);
                        if (qrow < p.N && col0 + c8 * 8 < p.N) bg[c8] = __ldg(reinterpret_cast<const uint4*>(bp + c8 * 8));
                    }
                }
                ok = warp_all(mbar_wait(&s_full[sbuf], (g >> 1) & 1, wc, 0x31));
                if (!ok) break;
                if ((warp & 3) == 0 && wg < 3) EVO_TL(p.status, 5 + wg, g, 1);
                EVO_TS(t_tile);
                tc_fence_after();
                uint32_t sv[2][16];
                tmem_ld16(tS, sv[0]);

                ok = warp_all(mbar_wait(&kv_full[st], (g / ST) & 1, wc, 0x32));
                if (!ok) break;
                uint32_t dep = 0;      // data the release of the stage must wait for
                {
                    // this warp's copy of the mask row slice: bf16 -> fp32 * log2e, -inf past N
                    if constexpr (CW == 64) {
                        const uint32_t mraw = sb + C::ST_MASK + 2 * CW * wg + 4 * lane;      // two bf16 per lane
                        uint32_t mw;
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(mw) : "r"(mraw));
                        dep = mw;
                        const int c = j * TILE + CW * wg + 2 * lane;
                        const float m0 = (c < p.N) ? bf16_lo(mw) * LOG2E : -INFINITY;
                        const float m1 = (c + 1 < p.N) ? bf16_hi(mw) * LOG2E : -INFINITY;
                        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(aWmask + 8 * lane), "f"(m0), "f"(m1) : "memory");
                    } else {
                        const uint32_t mraw = sb + C::ST_MASK + 2 * CW * wg + 2 * lane;      // one bf16 per lane
                        uint16_t mw;
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(mw) : "r"(mraw));
                        dep = mw;
                        const int c = j * TILE + CW * wg + lane;
                        const float m0 = (c < p.N) ? __uint_as_float(static_cast<uint32_t>(mw) << 16) * LOG2E : -INFINITY;
                        asm volatile("st.shared.f32 [%0], %1;" ::"r"(aWmask + 4 * lane), "f"(m0) : "memory");
                    }
                    __syncwarp();
                }
                // x = S*c1 + (bias*log2e + mask*log2e), in chunks of 16 columns; the tensor-memory
                // load of chunk ch+1 is in flight during the arithmetic of chunk ch
                float2 x2[CW / 2];
                float tmx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains: ILP
                const uint32_t sbias = sb + C::ST_BIAS + bias_sub;
#pragma unroll
                for (int ch = 0; ch < CW / 16; ++ch) {
                    const int cb = ch & 1;
                    tmem_wait_ld();
                    if (ch + 1 < CW / 16) {
                        tmem_ld16(tS + 16 * (ch + 1), sv[cb ^ 1]);
                    } else if (!C::WIDE) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&s_free[sbuf]);
                    }
                    uint4 b0, b1;
                    if constexpr (C::WIDE) {
                        b0 = bg[2 * ch];
                        b1 = bg[2 * ch + 1];
                    } else {
                        b0 = lds128(sbias + swz_off<128>(row, bias_c0 + 2 * ch));
                        b1 = lds128(sbias + swz_off<128>(row, bias_c0 + 2 * ch + 1));
                        dep ^= b0.x ^ b1.x;
                    }
                    const uint32_t bw[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                    float2 mm[8];
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const float4 mv = lds128f(aWmask + 64 * ch + 16 * q4);
                        mm[2 * q4] = make_float2(mv.x, mv.y);
                        mm[2 * q4 + 1] = make_float2(mv.z, mv.w);
                    }
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const float2 t2 = ffma2(bf16x2_f2(bw[k]), l2e2, mm[k]);
                        const float2 xx = ffma2(u2f2(sv[cb][2 * k], sv[cb][2 * k + 1]), c1x2, t2);
                        x2[ch * 8 + k] = xx;
                        tmx[k & 3] = fmax3(tmx[k & 3], xx.x, xx.y);
                    }
                }
                mbar_release_after_loads(&kv_empty[st], dep, scratch_w);      // bias tile and mask row are read
                if ((warp & 3) == 0 && wg < 3) EVO_TL(p.status, 5 + wg, g, 2);

                const float tmax = fmaxf(fmaxf(tmx[0], tmx[1]), fmaxf(tmx[2], tmx[3]));
                const float m_new = fmaxf(m_used, tmax);
                // When the running maximum rises (by more than EVO_FWD_LAZY), the accumulator in
                // tensor memory and the row sum are rescaled; otherwise the tensor core simply keeps
                // accumulating into the same tile.
                const bool need = (j > 0) && (m_new - m_used > EVO_FWD_LAZY);
                const float m_old = m_used;
                if (j == 0 || need) m_used = m_new;
                const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
                // The exp2 pass loads the special-function unit, the passes around it the other pipes.
                // Left alone the groups run in lockstep, all in the same pass at the same time.  At
                // D = 32 the two halves of the groups take turns instead: the first half runs the exp2
                // pass of tile g, then the second half runs its own, while the other half is in the
                // fused-multiply-add pass of its next tile or in its epilogue.  The first half waits
                // for the second half's pass of the previous tile, the second for the first's pass of
                // this tile.  (At D = 64 taking turns measured 7 % slower: 0.736 against 0.686 ms at B=1, S=256, N=1024, H=4.)
#ifdef EVO_FWD_NO_PINGPONG
                constexpr bool PINGPONG = false;
#else
                constexpr bool PINGPONG = (DH == 32);
#endif
                const int half = wg / (NG / 2);
                if (PINGPONG && (half == 1 || g > 0)) {
                    ok = warp_all(mbar_wait(&xu_done[half ^ 1], (half == 1 ? g : g - 1) & 1, wc, 0x38));
                    if (!ok) break;
                }
                // P = exp2(x - m), packed to bf16 pairs; row sum in two packed chains
                uint32_t pk[CW / 2];
                float rsum;
                {
                    const float2 nm2 = make_float2(-m_safe, -m_safe);
                    float2 rs[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
                    for (int c = 0; c < CW / 2; ++c) {
                        const float2 d2 = fadd2(x2[c], nm2);
                        const float2 p2 = make_float2(ex2(d2.x), ex2(d2.y));
                        rs[c & 1] = fadd2(rs[c & 1], p2);
                        pk[c] = pack_bf16(p2.x, p2.y);
                    }
                    rsum = (rs[0].x + rs[0].y) + (rs[1].x + rs[1].y);
                }
                if (PINGPONG) {
                    // hand the unit over; the store orders the arrive behind the last exp2 of the pass
                    __syncwarp();
                    if (lane == 0) {
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(scratch_w), "r"(pk[CW / 2 - 1]) : "memory");
                        mbar_arrive(&xu_done[half]);
                    }
                }

                // The P columns in tensor memory are free, and the accumulator may be rescaled, once
                // the previous tile's PV MMA is done.
                if ((warp & 3) == 0 && wg < 3) EVO_TL(p.status, 5 + wg, g, 3);
                if (g > 0) {
                    ok = warp_all(mbar_wait(&pv_full[wg], (g - 1) & 1, wc, 0x33));
                    if (!ok) break;
                    tc_fence_after();
                }
                if ((warp & 3) == 0 && wg < 3) EVO_TL(p.status, 5 + wg, g, 4);
                if (__any_sync(0xffffffffu, need)) {
                    // rescale this group's accumulator (lanes that need nothing scale by 1)
                    const float alpha = need ? ex2(m_old - m_safe) : 1.0f;
                    const float2 a2 = make_float2(alpha, alpha);
#pragma unroll
                    for (int c = 0; c < DH / 32; ++c) {
                        uint32_t r[32];
                        tmem_ld32(lane_base + C::TMEM_PV + wg * DH + c * 32, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const float2 v2 = fmul2(u2f2(r[i], r[i + 1]), a2);
                            r[i] = __float_as_uint(v2.x);
                            r[i + 1] = __float_as_uint(v2.y);
                        }
                        tmem_st32(lane_base + C::TMEM_PV + wg * DH + c * 32, r);
                    }
                    l *= alpha;
                }
                l += rsum;
                // P (bf16 pairs) into this group's columns of tensor memory
                if constexpr (CW == 64) tmem_st32(lane_base + C::p_col(wg, g), pk);
                else tmem_st16(lane_base + C::p_col(wg, g), pk);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_ready[wg]);
                if ((warp & 3) == 0 && wg < 3) EVO_TL(p.status, 5 + wg, g, 5);
                EVO_TE(t_tile, p.status, 0x78);
            }
            if (!ok) break;
            // publish this group's (m, l) of the item for the other groups' epilogues
            asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(aXch + (((it & 1) * NG + wg) * 128 + row) * 8),
                         "f"(m_used), "f"(l) : "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&xch_ready[(it & 1) * NG + wg]);
        }
    }

    if (tid == 0) EVO_TE(t_kernel, p.status, 0x7e);
    tc_fence_before();
    __syncthreads();
    EVO_TRACE_FLUSH(p.status);
    if (warp == W_S) tmem_dealloc(tmem, C::TMEM_COLS);
}

#ifndef EVO_FWD_NG32
#define EVO_FWD_NG32 2
#endif

// lay_in: q, k, v; lay: the output side (o, o_resid, gate, o_gated)
template <int DH, int NG>
static int launch_fwd(const EvoDims* d, const ActLayout& lay_in, const ActLayout& lay, const void* q, const void* k, const void* v,
                      const void* bias, const void* mask, const void* gate, void* o, void* o_gated, void* o_resid,
                      float* lse, float scale, cudaStream_t st) {
    using C = FwdCfg<DH, NG>;
    const int BS = d->B * d->S;
    const int QT = (d->N + TILE - 1) / TILE;

    CUtensorMap tq, tk, tv, tb, to;
    int rc;
    const int Dt = d->D;          // 16 on the D = 32 kernel: boxes of 32 columns over tensors of 16
    if ((rc = make_tmap_qkv(&tq, q, BS, d->N, d->H, Dt, TILE, lay_in, RowTile<DH>::BOX_D))) return rc;
    if ((rc = make_tmap_qkv(&tk, k, BS, d->N, d->H, Dt, TILE, lay_in, RowTile<DH>::BOX_D))) return rc;
    if ((rc = make_tmap_qkv(&tv, v, BS, d->N, d->H, Dt, TILE, lay_in, RowTile<DH>::BOX_D))) return rc;
    if ((rc = make_tmap_bias(&tb, bias, d->B, d->H, d->N))) return rc;
    if ((rc = make_tmap_qkv(&to, o, BS, d->N, d->H, Dt, TILE, lay, RowTile<DH>::BOX_D))) return rc;

    FwdParams p;
    p.B = d->B; p.S = d->S; p.N = d->N; p.H = d->H;
    p.Dt = Dt;
    p.KB = (Dt + 15) / 16;
    p.QT = QT;
    p.total_items = BS * QT * d->H;
    p.c1 = ((scale > 0.f) ? scale : 1.0f / sqrtf(static_cast<float>(Dt))) * LOG2E;
    p.mask = static_cast<const __nv_bfloat16*>(mask);
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.lse = lse;
    p.o_resid = static_cast<__nv_bfloat16*>(o_resid);
    p.gate = static_cast<const __nv_bfloat16*>(gate);
    p.o_gated = static_cast<__nv_bfloat16*>(o_gated);
    p.lay = lay;
    p.status = status_word();
    if (!p.status) return EVO_ERR_CUDA;

    int sms = 0;
    if ((rc = sm_count(&sms))) return rc;
    const ActLayout cl = contiguous_layout(d->N, d->H, DH);
    const bool strided = (lay.row != cl.row || lay.n != cl.n || lay.h != cl.h);
    auto kernel = gate ? (strided ? evo_fwd_kernel<DH, true, NG, true> : evo_fwd_kernel<DH, false, NG, true>)
                       : (strided ? evo_fwd_kernel<DH, true, NG, false> : evo_fwd_kernel<DH, false, NG, false>);
    if ((rc = set_max_smem_once(reinterpret_cast<const void*>(kernel), static_cast<int>(C::SMEM_BYTES))))
        return rc;
    const int grid = p.total_items < sms ? p.total_items : sms;
    prof_begin(0, st);
    kernel<<<grid, C::THREADS, C::SMEM_BYTES, st>>>(tq, tk, tv, tb, to, p);
    prof_end(0, st);
    return cuda_err(cudaGetLastError());
}

}  // namespace evo

extern "C" int evo_fwd(const EvoDims* dims, const void* q, const void* k, const void* v,
                       const void* pair_bias, const void* res_mask, void* o, void* o_resid, float* lse,
                       float scale, void* stream) {
    return evo_fwd_gated(dims, nullptr, q, k, v, pair_bias, res_mask, nullptr, o, nullptr, o_resid, lse, scale, stream);
}

extern "C" int evo_fwd_strided(const EvoDims* dims, const EvoStrides* strides, const void* q, const void* k,
                               const void* v, const void* pair_bias, const void* res_mask, void* o,
                               void* o_resid, float* lse, float scale, void* stream) {
    return evo_fwd_gated(dims, strides, q, k, v, pair_bias, res_mask, nullptr, o, nullptr, o_resid, lse, scale, stream);
}

extern "C" int evo_fwd_gated(const EvoDims* dims, const EvoStrides* strides, const void* q, const void* k,
                             const void* v, const void* pair_bias, const void* res_mask, const void* gate,
                             void* o, void* o_gated, void* o_resid, float* lse, float scale, void* stream) {
    return evo_fwd_views(dims, strides, strides, q, k, v, pair_bias, res_mask, gate, o, o_gated, o_resid, lse, scale,
                         stream);
}

extern "C" int evo_fwd_views(const EvoDims* dims, const EvoStrides* s_qkv, const EvoStrides* s_out, const void* q,
                             const void* k, const void* v, const void* pair_bias, const void* res_mask,
                             const void* gate, void* o, void* o_gated, void* o_resid, float* lse, float scale,
                             void* stream) {
    int rc = evo::check_dims(dims);
    if (rc) return rc;
    evo::ActLayout lay, lay_in;
    if ((rc = evo::layout_from_strides(dims, s_qkv, &lay_in))) return rc;
    if ((rc = evo::layout_from_strides(dims, s_out, &lay))) return rc;
    if (!q || !k || !v || !pair_bias || !res_mask || !o || !lse) return EVO_ERR_NULL_PTR;
    if ((gate == nullptr) != (o_gated == nullptr)) return EVO_ERR_NULL_PTR;
    const uintptr_t all = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                          reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(pair_bias) |
                          reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(o_resid) |
                          reinterpret_cast<uintptr_t>(res_mask) | reinterpret_cast<uintptr_t>(gate) |
                          reinterpret_cast<uintptr_t>(o_gated);
    if (all & 15u) return EVO_ERR_ALIGNMENT;
    if ((rc = evo::ensure_context())) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dims->D <= 32)
        return evo::launch_fwd<32, EVO_FWD_NG32>(dims, lay_in, lay, q, k, v, pair_bias, res_mask, gate, o, o_gated,
                                                 o_resid, lse, scale, st);
    if (dims->D <= 64)
        return evo::launch_fwd<64, 2>(dims, lay_in, lay, q, k, v, pair_bias, res_mask, gate, o, o_gated, o_resid, lse,
                                      scale, st);
    return evo::launch_fwd<128, 2>(dims, lay_in, lay, q, k, v, pair_bias, res_mask, gate, o, o_gated, o_resid, lse,
                                   scale, st);
}
