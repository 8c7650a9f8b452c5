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
// Four launches on one stream:
//   1. bwd_prep_kernel    delta and the extra tiles through which the main kernels add
//                         (mask - LSE) / scale to S and -delta to dP inside the tensor
//                         core (evo_tiles.cuh, "EXTRA TILE"), padded to whole tiles so
//                         the main kernels need no edge predicates
//   2. evo_dbias_kernel   dBias (evo_dbias.cu): one CTA per pair-bias tile keeps its
//                         sum over the S rows in registers, no reduction traffic
//   3. evo_bwd_kernel     dQ, dK, dV (below)
//   4. cvt_dq_kernel      fp32 dQ accumulator -> bf16 dQ in the caller layout
//
// evo_bwd_kernel: one persistent CTA per SM walks items (chunk of RC consecutive
// S rows, head h, kv tile j of 128 residues); per item it walks steps
// (q tile i, row r of the chunk), r innermost, so that one pair-bias tile serves
// RC steps.  dK/dV of every row of the chunk stay in tensor memory for the item.
//
//   warps 0-3, 4-7     two compute groups; group g owns kv columns 64g..64g+63
//                      (thread = one q row).  Per step: P = exp2(S' c1 + bias log2e)
//                      and dS = P dP' from the two accumulators, kept packed in
//                      registers until the previous step's dV/dK/dQ MMAs have
//                      finished reading the P/dS tiles, then written to shared
//                      memory as MMA operands.
//   warps 8-11 (drain) warp w owns tensor-memory lanes 32(w-8)..: after every step
//                      it stages its 32 rows of dQ in its own shared-memory slot and
//                      issues a TMA reduce-add (fp32) for them; after an item, dK/dV
//                      go out as bf16 stores.  None of this is on the compute groups'
//                      path.
//   warp 12 (producer) TMA per step: Q, dO tiles and the extra tile of the q rows; K, V
//                      tiles and the extra tile of the kv rows per step (D=32) or per
//                      item (D>=64); the pair-bias tile per q tile (D<=64)
//   warps 13, 14, 15   tcgen05.mma issuers, one chain family each, so that no chain
//                      queues behind another's issue: S' = Q K^T + extra block and
//                      dP' = dO V^T + extra block of the next step (13);
//                      dV += P^T dO and dK += dS^T Q (14); dQ = dS K (15).  Each warp
//                      runs its loop with all lanes and elects one lane to issue.
#include "evo_dbias.cuh"
#include "evo_host.cuh"
#include "evo_ptx.cuh"
#include "evo_tiles.cuh"

#include <mutex>


namespace evo {

// 4 warpgroups: 2 compute, drain, (producer, mma, 2 idle warps)
constexpr int BWD_THREADS = 512;
constexpr int BWD_WARP_DRAIN = 8, BWD_WARP_PRODUCER = 12, BWD_WARP_MMA = 13;   // 13, 14, 15: mma issuers
constexpr uint32_t BWD_TMEM_COLS = 512;
// setmaxnreg budgets of the compute warpgroups and of the others, by head dim.  Measured (dQ/dK/dV
// kernel): D=32 (B=1, S=512, N=384, H=8) 168/88 0.474 ms, 176/80 0.471, 184/72 0.483, 160/96 0.478;
// D=64 (B=1, S=256, N=1024, H=4) 168/88 1.297 ms, 176/80 1.321, 184/72 1.288, 160/96 1.353.
template <int DH> constexpr int BWD_REGS_COMPUTE = (DH == 64) ? 184 : 176;
template <int DH> constexpr int BWD_REGS_OTHER = 256 - BWD_REGS_COMPUTE<DH>;
// the CTA's register pool is the launch count (cap for 512 threads: 128) times the threads;
// a setmaxnreg increase that the pool cannot satisfy blocks for ever
static_assert(BWD_REGS_COMPUTE<32> * 256 + BWD_REGS_OTHER<32> * 256 <= 128 * BWD_THREADS, "register pool");

template <int DH>
struct BwdCfg {
    static constexpr int RC = (DH == 32) ? 3 : 1;     // S rows per chunk
#ifndef EVO_BWD_QS32
#define EVO_BWD_QS32 3
#endif
    static constexpr int QS = (DH == 32) ? EVO_BWD_QS32 : (DH == 64 ? 2 : 1);     // load stages
    // D=32: K/V travel with every step's stage; D>=64: one resident K/V buffer per item
    static constexpr bool KV_RESIDENT = (DH >= 64);
    // D=128 is short of shared and tensor memory: one load stage, the bias slice of a thread read
    // straight from global memory (no staged tile), and ONE dQ accumulator that shares its tensor
    // memory columns with S' (S' of step n+1 is issued once dQ of step n is drained).
    static constexpr bool BIAS_STAGED = (DH <= 64);
    static constexpr int DQ_BUFS = (DH <= 64) ? 2 : 1;
    static constexpr int HALF = DH / 2;               // head-dim columns drained per group
    static constexpr uint32_t ROWT = RowTile<DH>::BYTES;
    // one stage: Q, dO [, K, V] tiles, then the extra tile of the q rows [and of the kv rows]
    static constexpr uint32_t ST_Q = 0, ST_DO = ROWT;
    static constexpr uint32_t ST_K = 2 * ROWT, ST_V = 3 * ROWT;            // streaming only
    static constexpr uint32_t ST_TILES = KV_RESIDENT ? 2 : 4;
    static constexpr uint32_t ST_XQ = ST_TILES * ROWT, ST_XK = ST_XQ + XT_BYTES;
    static constexpr uint32_t STAGE_TX = ST_TILES * ROWT + (KV_RESIDENT ? 1 : 2) * XT_BYTES;
    static constexpr uint32_t STAGE_STRIDE = ST_TILES * ROWT + 2 * XT_BYTES;
    // resident K/V buffer: K[RC], V[RC], extra tiles of the kv rows [RC]
    static constexpr uint32_t KV_BYTES = KV_RESIDENT ? (2 * RC * ROWT + RC * XT_BYTES) : 0;
    static constexpr uint32_t KV_TX = 2 * ROWT + XT_BYTES;                  // per row of the chunk
    static constexpr uint32_t OFF_STAGE = 0;
    static constexpr uint32_t OFF_KV = OFF_STAGE + QS * STAGE_STRIDE;
    static constexpr uint32_t OFF_BIAS = OFF_KV + KV_BYTES;
    static constexpr uint32_t OFF_P = OFF_BIAS + (BIAS_STAGED ? SQ_BYTES : 0);
    static constexpr uint32_t OFF_DS = OFF_P + SQ_BYTES;
    // per drain warp: dQ slot [32 rows][32 fp32]
    static constexpr uint32_t WQ_BYTES = 32 * 32 * 4;
    static constexpr uint32_t OFF_WSTG = OFF_DS + SQ_BYTES;
    // constant extra tiles, above every tile that refers to the zero tile
    static constexpr uint32_t OFF_XDP = OFF_WSTG + 4 * WQ_BYTES;            // column selector of -delta
    static constexpr uint32_t OFF_ZERO = OFF_XDP + XT_BYTES;
    static constexpr uint32_t OFF_BARS = OFF_ZERO + XT_BYTES;
    static constexpr uint32_t NUM_BARS = 2 * QS + 2 + 2 + 7 + RC + 2;
    static constexpr uint32_t OFF_MISC = OFF_BARS + NUM_BARS * 8;
    static constexpr uint32_t SMEM_BYTES = OFF_MISC + 16 + 1024;            // + alignment slack
    static constexpr uint32_t TMEM_S = 0;
    static constexpr uint32_t TMEM_DP = 128;
    static constexpr uint32_t TMEM_DQ = (DQ_BUFS == 2) ? 256 : TMEM_S;      // DQ_BUFS accumulators, + (step % DQ_BUFS)*DH
    static constexpr uint32_t TMEM_DKV = (DQ_BUFS == 2) ? 256 + 2 * DH : 256;   // + r*2*DH (dK), + DH (dV)
    static_assert(TMEM_DKV + RC * 2 * DH <= BWD_TMEM_COLS, "tensor memory budget");
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
    static_assert(OFF_KV % 1024 == 0 && OFF_BIAS % 1024 == 0 && WQ_BYTES % 1024 == 0, "tile alignment");
};

struct BwdParams {
    int B, S, N, H;
    int Dt;          // true head dim (16 runs on the D = 32 kernel: loads zero-filled, stores clipped)
    int KB;          // contraction blocks of 16 head-dim columns that hold data: ceil(Dt / 16)
    int NT;          // tiles per row: ceil(N / 128)
    int NTP;         // NT * 128
    int CPB;         // chunks per batch: ceil(S / RC)
    int total_items; // B * CPB * H * NT
    float scale;     // softmax scale
    float c1;        // scale * log2(e)
    const __nv_bfloat16* xq;   // [B*S][H][NTP][8] extra tiles of the q rows  (bwd_prep_kernel)
    const __nv_bfloat16* xk;   // [B*S][NTP][8]    extra tiles of the kv rows
    const __nv_bfloat16* bias; // [B][H][N][N] (read directly when the bias tile is not staged)
    float* dbias;              // [B][H][N][N] (written by this kernel only when S = 1)
    __nv_bfloat16* dk;    // activation layout `lay`
    __nv_bfloat16* dv;
    ActLayout lay;        // element strides of the activation tensors
    unsigned int* status;
};

struct BwdItem {
    int b, bs0, nr, h, j;
};

// DBIAS_HERE (S = 1 only): dBias is dS itself, no sum over rows, so the compute groups store their
// fp32 dS straight to d_pair_bias and the dBias kernel (which would recompute S and dP for one step
// per item) is not launched.
template <int DH, bool DBIAS_HERE>
__global__ void __launch_bounds__(BWD_THREADS, 1)
evo_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
               const __grid_constant__ CUtensorMap tm_bias, const __grid_constant__ CUtensorMap tm_dq,
               const BwdParams p) {
    using C = BwdCfg<DH>;
    using RT = RowTile<DH>;
    using RD = RowDesc<DH>;
    constexpr int RC = C::RC, QS = C::QS;
    constexpr bool KVR = C::KV_RESIDENT;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BARS);
    uint64_t* st_full = bars;                  // [QS]
    uint64_t* st_empty = st_full + QS;         // [QS]
    uint64_t* kv_full = st_empty + QS;         // resident K/V only
    uint64_t* kv_empty = kv_full + 1;
    uint64_t* bias_full = kv_empty + 1;
    uint64_t* bias_empty = bias_full + 1;
    uint64_t* sdp_full = bias_empty + 1;
    uint64_t* sdp_free = sdp_full + 1;
    uint64_t* pds_ready = sdp_free + 1;
    uint64_t* dq_full = pds_ready + 1;         // [2]
    uint64_t* dq_free = dq_full + 2;           // [2]
    uint64_t* dkv_free = dq_free + 2;          // [RC]: accumulators of row r of the chunk are read out
    uint64_t* tail_done = dkv_free + RC;       // [2] by step parity: both tail issuers' MMAs of a step are complete
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
        mbar_init(kv_full, 1);
        mbar_init(kv_empty, 2);
        for (int i = 0; i < 2; ++i) mbar_init(&tail_done[i], 2);
        mbar_init(bias_full, 1);
        mbar_init(bias_empty, 8);
        mbar_init(sdp_full, 1);
        mbar_init(sdp_free, 8);
        mbar_init(pds_ready, 8);
        for (int i = 0; i < 2; ++i) { mbar_init(&dq_full[i], 1); mbar_init(&dq_free[i], 4); }
        for (int i = 0; i < RC; ++i) mbar_init(&dkv_free[i], 4);
        fence_mbar_init();
        fence_async_smem();
    }
    if (warp == BWD_WARP_MMA) {
        tmem_alloc(tmem_slot, BWD_TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == BWD_WARP_PRODUCER && lane == 0) {
        prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); prefetch_tmap(&tm_do);
        prefetch_tmap(&tm_bias); prefetch_tmap(&tm_dq);
    }
    // constant extra tiles: row n of the -delta selector is (0,0,0,0,1,1,0,0); the zero tile
    if (tid < 128) {
        *reinterpret_cast<uint4*>(smem + C::OFF_XDP + tid * 16) = make_uint4(0u, 0u, 0x3f803f80u, 0u);
        *reinterpret_cast<uint4*>(smem + C::OFF_ZERO + tid * 16) = make_uint4(0u, 0u, 0u, 0u);
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

    if (warp >= BWD_WARP_DRAIN) {
        reg_dec<BWD_REGS_OTHER<DH>>();
        if (warp == BWD_WARP_PRODUCER && lane == 0) {
            // ------------------------------ producer ------------------------------
            bool ok = true;
            int gs = 0, gb = 0;
            for (int it = 0; it < n_items && ok; ++it) {
                const BwdItem x = decode(it);
                const int nsteps = NT * x.nr;
                if (KVR) {
                    if (it > 0) ok = mbar_wait(kv_empty, (it - 1) & 1, wc, 0x40);
                    if (!ok) break;
                    uint8_t* kvb = smem + C::OFF_KV;
                    mbar_arrive_expect_tx(kv_full, x.nr * C::KV_TX);
                    for (int r = 0; r < x.nr; ++r) {
                        tma_load_row_tile<DH>(kvb + r * C::ROWT, &tm_k, kv_full, x.h, x.j * TILE, x.bs0 + r);
                        tma_load_row_tile<DH>(kvb + (RC + r) * C::ROWT, &tm_v, kv_full, x.h, x.j * TILE, x.bs0 + r);
                        bulk_load(kvb + 2 * RC * C::ROWT + r * XT_BYTES,
                                  p.xk + (static_cast<size_t>(x.bs0 + r) * p.NTP + x.j * TILE) * 8, XT_BYTES, kv_full);
                    }
                }
                for (int n = 0; n < nsteps && ok; ++n, ++gs) {
                    const int i = n / x.nr, r = n - i * x.nr;
                    const int st = gs % QS;
                    if (C::BIAS_STAGED && r == 0) {
                        if (gb > 0) ok = mbar_wait(bias_empty, (gb - 1) & 1, wc, 0x41);
                        if (!ok) break;
                        mbar_arrive_expect_tx(bias_full, SQ_BYTES);
                        tma_load_4d(smem + C::OFF_BIAS, &tm_bias, bias_full, x.j * TILE, i * TILE, x.h, x.b);
                        tma_load_4d(smem + C::OFF_BIAS + SQ_SUB_BYTES, &tm_bias, bias_full, x.j * TILE + 64,
                                    i * TILE, x.h, x.b);
                        ++gb;
                    }
                    if (gs >= QS) ok = mbar_wait(&st_empty[st], ((gs / QS) - 1) & 1, wc, 0x42);
                    if (!ok) break;
                    const int bs = x.bs0 + r;
                    uint8_t* sb = smem + C::OFF_STAGE + st * C::STAGE_STRIDE;
                    mbar_arrive_expect_tx(&st_full[st], C::STAGE_TX);
                    tma_load_row_tile<DH>(sb + C::ST_Q, &tm_q, &st_full[st], x.h, i * TILE, bs);
                    tma_load_row_tile<DH>(sb + C::ST_DO, &tm_do, &st_full[st], x.h, i * TILE, bs);
                    if (!KVR) {
                        tma_load_row_tile<DH>(sb + C::ST_K, &tm_k, &st_full[st], x.h, x.j * TILE, bs);
                        tma_load_row_tile<DH>(sb + C::ST_V, &tm_v, &st_full[st], x.h, x.j * TILE, bs);
                        bulk_load(sb + C::ST_XK, p.xk + (static_cast<size_t>(bs) * p.NTP + x.j * TILE) * 8, XT_BYTES,
                                  &st_full[st]);
                    }
                    const size_t ro = (static_cast<size_t>(bs) * p.H + x.h) * p.NTP + i * TILE;
                    bulk_load(sb + C::ST_XQ, p.xq + ro * 8, XT_BYTES, &st_full[st]);
                }
            }
            // Drain: the most recent loads have landed before the CTA exits.
            for (int k = (gs > QS ? gs - QS : 0); k < gs; ++k)
                (void)mbar_wait(&st_full[k % QS], (k / QS) & 1, wc, 0x43);
            if (gb > 0) (void)mbar_wait(bias_full, (gb - 1) & 1, wc, 0x44);
            if (KVR && n_items > 0) (void)mbar_wait(kv_full, (n_items - 1) & 1, wc, 0x45);
        } else if (warp >= BWD_WARP_MMA) {
            // ------------------------------ mma issuers ------------------------------
            // Three warps, one chain family each, so that no chain queues behind another one's
            // issue: warp 13 issues S' and dP' of the next step as soon as the compute groups have
            // read the previous pair, warp 14 issues dV += P^T dO and dK += dS^T Q, warp 15 issues
            // dQ = dS K.  Each warp runs its loop with all lanes (uniform control flow: operand
            // descriptors stay in uniform registers) and elects one lane to issue.
            constexpr uint32_t IDESC_SDP = make_idesc_bf16(128, 128, 0, 0);
            // N = the head-dim columns that hold data (the rest of a wider kernel's tile is zero fill)
            const uint32_t IDESC_DKV = make_idesc_bf16(128, 16 * p.KB, 1, 1);
            const uint32_t IDESC_DQ = make_idesc_bf16(128, 16 * p.KB, 0, 1);
            const uint32_t aSt = smem_u32(smem + C::OFF_STAGE), aKV = smem_u32(smem + C::OFF_KV);
            const uint32_t aZero = smem_u32(smem + C::OFF_ZERO);
            const int role = warp - BWD_WARP_MMA;          // 0: S/dP, 1: dV/dK, 2: dQ
            bool ok = true;
            int gs = 0;
            for (int it = 0; it < n_items && ok; ++it) {
                const BwdItem x = decode(it);
                const int nsteps = NT * x.nr;
                int i = 0, r = 0;
                for (int n = 0; n < nsteps && ok; ++n, ++gs) {
                    const int st = gs % QS;
                    const uint32_t sb = aSt + st * C::STAGE_STRIDE;
                    const uint32_t k_tile = KVR ? aKV + r * C::ROWT : sb + C::ST_K;
                    if (role == 0) {
                        ok = warp_all(mbar_wait(&st_full[st], (gs / QS) & 1, wc, 0x50));
                        if (ok && KVR && n == 0) ok = warp_all(mbar_wait(kv_full, it & 1, wc, 0x51));
                        if (ok && gs > 0) ok = warp_all(mbar_wait(sdp_free, (gs - 1) & 1, wc, 0x52));
                        // S' shares its columns with the single dQ accumulator: the previous step's dQ is drained
                        if (ok && C::DQ_BUFS == 1 && gs > 0) ok = warp_all(mbar_wait(&dq_free[0], (gs - 1) & 1, wc, 0x56));
                        if (!ok) break;
                        tc_fence_after();
                        if (elect_one()) {
                            const uint32_t v_tile = KVR ? aKV + (RC + r) * C::ROWT : sb + C::ST_V;
                            const uint32_t q_lo = RD::kmajor_lo(sb + C::ST_Q), do_lo = RD::kmajor_lo(sb + C::ST_DO);
                            const uint32_t k_lo = RD::kmajor_lo(k_tile), v_lo = RD::kmajor_lo(v_tile);
#pragma unroll
                            for (int kk = 0; kk < RT::KBLOCKS; ++kk) {
                                if (kk >= p.KB) continue;      // zero-filled blocks past the true head dim
                                umma_ss(tmem + C::TMEM_S, RD::kmajor(q_lo, kk), RD::kmajor(k_lo, kk), IDESC_SDP, kk > 0);
                                umma_ss(tmem + C::TMEM_DP, RD::kmajor(do_lo, kk), RD::kmajor(v_lo, kk), IDESC_SDP, kk > 0);
                            }
                            // + (mask - LSE) / scale on S, - delta on dP: the extra contraction block
                            const uint64_t d_xq = xt_desc(sb + C::ST_XQ, aZero);
                            const uint32_t xk_addr = KVR ? aKV + 2 * RC * C::ROWT + r * XT_BYTES : sb + C::ST_XK;
                            umma_ss(tmem + C::TMEM_S, d_xq, xt_desc(xk_addr, aZero), IDESC_SDP, 1u);
                            umma_ss(tmem + C::TMEM_DP, d_xq, xt_desc(smem_u32(smem + C::OFF_XDP), aZero), IDESC_SDP, 1u);
                            umma_commit(sdp_full);
                        }
                        __syncwarp();
                    } else if (role == 1) {
                        ok = warp_all(mbar_wait(pds_ready, gs & 1, wc, 0x53));
                        // the first MMA into row r's dK/dV of an item overwrites them: the previous item's must be out
                        if (ok && i == 0 && it > 0) ok = warp_all(mbar_wait(&dkv_free[r], (it - 1) & 1, wc, 0x55));
                        if (!ok) break;
                        tc_fence_after();
                        if (elect_one()) {
                            const uint32_t p_mn_lo = SqDesc::mnmajor_lo(smem_u32(smem + C::OFF_P));
                            const uint32_t ds_mn_lo = SqDesc::mnmajor_lo(smem_u32(smem + C::OFF_DS));
                            const uint32_t q_lo = RD::mnmajor_lo(sb + C::ST_Q), do_lo = RD::mnmajor_lo(sb + C::ST_DO);
                            const uint32_t t_dk = tmem + C::TMEM_DKV + r * 2 * DH, t_dv = t_dk + DH;
                            const uint32_t acc = (i > 0) ? 1u : 0u;
#pragma unroll
                            for (int kk = 0; kk < 8; ++kk) {      // two interleaved chains
                                umma_ss(t_dv, SqDesc::mnmajor(p_mn_lo, kk), RD::mnmajor(do_lo, kk), IDESC_DKV, kk > 0 ? 1u : acc);
                                umma_ss(t_dk, SqDesc::mnmajor(ds_mn_lo, kk), RD::mnmajor(q_lo, kk), IDESC_DKV, kk > 0 ? 1u : acc);
                            }
                            umma_commit(&tail_done[gs & 1]);
                            umma_commit(&st_empty[st]);
                            if (KVR && n == nsteps - 1) umma_commit(kv_empty);
                        }
                        __syncwarp();
                    } else if (role == 2) {
                        ok = warp_all(mbar_wait(pds_ready, gs & 1, wc, 0x53));
                        if (ok && gs >= C::DQ_BUFS)
                            ok = warp_all(mbar_wait(&dq_free[gs % C::DQ_BUFS], ((gs / C::DQ_BUFS) - 1) & 1, wc, 0x54));
                        if (!ok) break;
                        tc_fence_after();
                        if (elect_one()) {
                            const uint32_t ds_k_lo = SqDesc::kmajor_lo(smem_u32(smem + C::OFF_DS));
                            const uint32_t k_lo = RD::mnmajor_lo(k_tile);
                            const uint32_t t_dq = tmem + C::TMEM_DQ + (gs % C::DQ_BUFS) * DH;
#pragma unroll
                            for (int kk = 0; kk < 8; ++kk)
                                umma_ss(t_dq, SqDesc::kmajor(ds_k_lo, kk), RD::mnmajor(k_lo, kk), IDESC_DQ, kk > 0);
                            umma_commit(&dq_full[gs % C::DQ_BUFS]);
                            umma_commit(&tail_done[gs & 1]);
                            umma_commit(&st_empty[st]);
                            if (KVR && n == nsteps - 1) umma_commit(kv_empty);
                        }
                        __syncwarp();
                    }
                    if (++r == x.nr) { r = 0; ++i; }
                }
            }
        } else if (warp < BWD_WARP_DRAIN + 4) {
            // ------------------------------ drain warps ------------------------------
            const int wrow0 = (warp & 3) * 32;   // tensor-memory lanes (tile rows) of this warp
            const uint32_t lane_base = tmem + (static_cast<uint32_t>(wrow0) << 16);
            uint8_t* wq = smem + C::OFF_WSTG + (warp & 3) * C::WQ_BYTES;
            bool ok = true;
            int gs = 0;
            for (int it = 0; it < n_items && ok; ++it) {
                const BwdItem x = decode(it);
                const int nsteps = NT * x.nr;
                int i = 0, r = 0;
                for (int n = 0; n < nsteps && ok; ++n, ++gs) {
                    const int b = gs % C::DQ_BUFS;
                    ok = warp_all(mbar_wait(&dq_full[b], (gs / C::DQ_BUFS) & 1, wc, 0x68));
                    if (!ok) break;
                    tc_fence_after();
                    // dQ of this step: tensor memory -> this warp's slot -> fp32 reduce-add
#pragma unroll
                    for (int rd = 0; rd < DH / 32; ++rd) {
                        float dqv[32];
                        tmem_ld_f32<32>(lane_base + C::TMEM_DQ + b * DH + rd * 32, dqv);
                        if (rd == DH / 32 - 1) {
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&dq_free[b]);
                        }
                        if (i * TILE + wrow0 < p.N && rd * 32 < p.Dt) {     // warp-uniform
                            // the slot is free once lane 0's earlier bulk operations have read it
                            if (lane == 0) tma_wait_group_read<0>();
                            __syncwarp();
#pragma unroll
                            for (int cc = 0; cc < 8; ++cc)
                                *reinterpret_cast<float4*>(wq + swz_off<128>(lane, cc)) =
                                    make_float4(dqv[cc * 4 + 0] * p.scale, dqv[cc * 4 + 1] * p.scale,
                                                dqv[cc * 4 + 2] * p.scale, dqv[cc * 4 + 3] * p.scale);
                            fence_async_smem();
                            __syncwarp();
                            if (lane == 0) {
                                tma_reduce_add_4d(&tm_dq, wq, rd * 32, x.h, i * TILE + wrow0, x.bs0 + r);
                                tma_commit_group();
                            }
                        }
                    }
                    if (n == nsteps - 1) {
                        ok = warp_all(mbar_wait(&tail_done[gs & 1], (gs >> 1) & 1, wc, 0x69));
                        if (!ok) break;
                        tc_fence_after();
                        // the item's last MMAs are done: dK/dV -> bf16 stores, row by row of the chunk;
                        // each row's accumulators are handed back as soon as they are read
                        const int kvrow = x.j * TILE + wrow0 + lane;
#pragma unroll
                        for (int rr = 0; rr < RC; ++rr) {
                            if (rr < x.nr) {
#pragma unroll
                                for (int t = 0; t < 2; ++t) {      // 0: dK, 1: dV
                                    const float sc = t ? 1.0f : p.scale;
                                    __nv_bfloat16* out = (t ? p.dv : p.dk) + (x.bs0 + rr) * p.lay.row +
                                                         kvrow * p.lay.n + x.h * p.lay.h;
#pragma unroll
                                    for (int hf = 0; hf < DH / 32; ++hf) {
                                        float v[32];
                                        tmem_ld_f32<32>(lane_base + C::TMEM_DKV + rr * 2 * DH + t * DH + hf * 32, v);
                                        if (kvrow < p.N) {
#pragma unroll
                                            for (int c8 = 0; c8 < 4; ++c8) {
                                                if (hf * 32 + c8 * 8 >= p.Dt) continue;
                                                uint4 u;
                                                u.x = pack_bf16(v[c8 * 8 + 0] * sc, v[c8 * 8 + 1] * sc);
                                                u.y = pack_bf16(v[c8 * 8 + 2] * sc, v[c8 * 8 + 3] * sc);
                                                u.z = pack_bf16(v[c8 * 8 + 4] * sc, v[c8 * 8 + 5] * sc);
                                                u.w = pack_bf16(v[c8 * 8 + 6] * sc, v[c8 * 8 + 7] * sc);
                                                *reinterpret_cast<uint4*>(out + hf * 32 + c8 * 8) = u;
                                            }
                                        }
                                    }
                                }
                            }
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&dkv_free[rr]);
                        }
                    }
                    if (++r == x.nr) { r = 0; ++i; }
                }
            }
            if (lane == 0) tma_wait_group<0>();
        }
    } else {
        reg_inc<BWD_REGS_COMPUTE<DH>>();
        // ------------------------------ compute groups ------------------------------
        const int wg = warp >> 2;            // kv columns 64*wg .. 64*wg+63 of the tile
        const int row = tid & 127;           // q row within the tile == TMEM lane
        const int wrow0 = (warp & 3) * 32;   // first tile row of this warp
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(wrow0) << 16);
        const uint32_t aP = smem_u32(smem + C::OFF_P) + wg * SQ_SUB_BYTES;
        const uint32_t aDS = smem_u32(smem + C::OFF_DS) + wg * SQ_SUB_BYTES;
        const uint32_t aBias = smem_u32(smem + C::OFF_BIAS) + wg * SQ_SUB_BYTES;
        const uint32_t scratch_w = smem_u32(tmem_slot + 2);       // a word nobody reads
        bool ok = true;
        int gs = 0, gb = 0;
        const float2 c1x2 = make_float2(p.c1, p.c1), l2e2 = make_float2(LOG2E, LOG2E);

        uint32_t bias_pk[32];                // this thread's 64 bias values (bf16 pairs)

        for (int it = 0; it < n_items && ok; ++it) {
            const BwdItem x = decode(it);
            const int nsteps = NT * x.nr;
            int r = 0;                       // row of the chunk, innermost
            for (int n = 0; n < nsteps && ok; ++n, ++gs) {
                if (!C::BIAS_STAGED && r == 0) {
                    // this thread's 64 bias values of q tile n / nr, straight from global memory,
                    // requested before the wait so that they arrive while the MMAs run
                    const int qrow = (n / x.nr) * TILE + row, col0 = x.j * TILE + 64 * wg;
                    const __nv_bfloat16* bp = p.bias + ((static_cast<size_t>(x.b) * p.H + x.h) * p.N + qrow) * p.N + col0;
#pragma unroll
                    for (int c8 = 0; c8 < 8; ++c8) {
                        uint4 bv = make_uint4(0u, 0u, 0u, 0u);
                        if (qrow < p.N && col0 + c8 * 8 < p.N) bv = __ldg(reinterpret_cast<const uint4*>(bp + c8 * 8));
                        bias_pk[c8 * 4 + 0] = bv.x; bias_pk[c8 * 4 + 1] = bv.y;
                        bias_pk[c8 * 4 + 2] = bv.z; bias_pk[c8 * 4 + 3] = bv.w;
                    }
                }
                ok = warp_all(mbar_wait(sdp_full, gs & 1, wc, 0x63));
                if (!ok) break;
                EVO_TS(t_cmp);
                if (C::BIAS_STAGED && r == 0) {
                    ok = warp_all(mbar_wait(bias_full, gb & 1, wc, 0x64));
                    if (!ok) break;
                    uint32_t dep = 0;
#pragma unroll
                    for (int c8 = 0; c8 < 8; ++c8) {
                        const uint4 bv = lds128(aBias + swz_off<128>(row, c8));
                        bias_pk[c8 * 4 + 0] = bv.x; bias_pk[c8 * 4 + 1] = bv.y;
                        bias_pk[c8 * 4 + 2] = bv.z; bias_pk[c8 * 4 + 3] = bv.w;
                        dep ^= bv.x;
                    }
                    mbar_release_after_loads(bias_empty, dep, scratch_w);     // the tile now lives in registers
                    ++gb;
                }

                // Per element: x = S' c1 + bias log2e (S' already carries mask and -LSE through the
                // extra contraction block), P = exp2(x), dS = P dP' (dP' already carries -delta).
                // Chunks of 16 columns; the tensor-memory loads of chunk ch+1 are in flight during
                // the arithmetic of chunk ch.
                uint32_t pkp[32], pkd[32];           // P and dS of this thread's 64 columns, bf16 pairs
                uint32_t sv[2][16], dv[2][16];
                tc_fence_after();
                tmem_ld16(lane_base + C::TMEM_S + 64 * wg, sv[0]);
                tmem_ld16(lane_base + C::TMEM_DP + 64 * wg, dv[0]);
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    const int cb = ch & 1;
                    tmem_wait_ld();
                    if (ch < 3) {
                        tmem_ld16(lane_base + C::TMEM_S + 64 * wg + 16 * (ch + 1), sv[cb ^ 1]);
                        tmem_ld16(lane_base + C::TMEM_DP + 64 * wg + 16 * (ch + 1), dv[cb ^ 1]);
                    } else {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(sdp_free);
                    }
                    float2 p2[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const float2 b2 = fmul2(bf16x2_f2(bias_pk[ch * 8 + k]), l2e2);
                        const float2 x2 = ffma2(u2f2(sv[cb][2 * k], sv[cb][2 * k + 1]), c1x2, b2);
                        p2[k] = make_float2(ex2(x2.x), ex2(x2.y));
                    }
                    float2 dsv[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const float2 ds2 = fmul2(p2[k], u2f2(dv[cb][2 * k], dv[cb][2 * k + 1]));
                        pkp[ch * 8 + k] = pack_bf16(p2[k].x, p2[k].y);
                        pkd[ch * 8 + k] = pack_bf16(ds2.x, ds2.y);
                        dsv[k] = ds2;
                    }
                    if constexpr (DBIAS_HERE) {
                        // one S row: this step's dS tile is the dBias tile (q tile n, kv tile j)
                        const int qrow = (n / x.nr) * TILE + row, c0 = x.j * TILE + 64 * wg + 16 * ch;
                        if (qrow < p.N) {
                            float* out = p.dbias + ((static_cast<size_t>(x.b) * p.H + x.h) * p.N + qrow) * p.N + c0;
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4)
                                if (c0 + q4 * 4 < p.N)
                                    *reinterpret_cast<float4*>(out + q4 * 4) =
                                        make_float4(dsv[2 * q4].x, dsv[2 * q4].y, dsv[2 * q4 + 1].x, dsv[2 * q4 + 1].y);
                        }
                    }
                }
                EVO_TE(t_cmp, p.status, 0x70);

                // the P / dS tiles are free once the previous step's dV/dK/dQ MMAs are done
                if (gs > 0) {
                    ok = warp_all(mbar_wait(&tail_done[(gs - 1) & 1], ((gs - 1) >> 1) & 1, wc, 0x61));
                    if (!ok) break;
                }
                EVO_TS(t_sts);
#pragma unroll
                for (int c8 = 0; c8 < 8; ++c8) {
                    const uint32_t off = swz_off<128>(row, c8);
                    sts128(aP + off, make_uint4(pkp[c8 * 4 + 0], pkp[c8 * 4 + 1], pkp[c8 * 4 + 2], pkp[c8 * 4 + 3]));
                    sts128(aDS + off, make_uint4(pkd[c8 * 4 + 0], pkd[c8 * 4 + 1], pkd[c8 * 4 + 2], pkd[c8 * 4 + 3]));
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(pds_ready);
                EVO_TE(t_sts, p.status, 0xb3);
                if (++r == x.nr) r = 0;
            }
        }
    }

    if (tid == 0) EVO_TE(t_kernel, p.status, 0x7f);
    tc_fence_before();
    __syncthreads();
    EVO_TRACE_FLUSH(p.status);
    if (warp == BWD_WARP_MMA) tmem_dealloc(tmem, BWD_TMEM_COLS);
}

// ---------------------------------------------------------------------------
// prep: delta = rowsum(dO o O) (replaces evo_bwd_prep_ker, tk_evoattention.cu:352-416),
// and the extra tiles through which the main kernels add every per-row and per-column
// term of the logits inside the tensor core (evo_tiles.cuh, "EXTRA TILE"):
//
//   xq [B*S][H][NTP][8] bf16, row q:  ( 1, 1, a_hi, a_lo, -d_hi, -d_lo, 0, 0 )   a = -LSE / scale
//   xk [B*S][NTP][8]    bf16, row kv: ( m_hi, m_lo, 1, 1, 0, 0, 0, 0 )           m = mask / scale
//
// so that  Q K^T + xq xk^T = Q K^T + (mask - LSE) / scale  (times scale*log2e: the base-2
// logit minus the base-2 LSE) and  dO V^T + xq (0,0,0,0,1,1,0,0)^T = dP - delta.
// Values are split into a bf16 head and a bf16 remainder (16 significant bits).  Rows
// past N (padding up to whole tiles, NTP = tiles * 128) get a = m = -1e30: finite, so
// that a product with a zero of the other tile stays zero, and far below any logit.
// With o_resid (the bf16 rounding residual of O written by the forward), delta
// uses O to about 16 bits instead of 8: the rounding of O otherwise puts an
// error of order 2^-9 |dO||O| on every dS, which adds up over the S rows of dBias.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t split_bf16(float v) {
    // (head, remainder) as a bf16 pair, head in the low half
    v = fminf(fmaxf(v, -1e30f), 1e30f);
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    const __nv_bfloat16 lo = __float2bfloat16_rn(v - __bfloat162float(hi));
    return static_cast<uint32_t>(__bfloat16_as_ushort(hi)) | (static_cast<uint32_t>(__bfloat16_as_ushort(lo)) << 16);
}

// With a gate (evo_bwd_gated) d_o is the gradient of the GATED output: the kernel then also forms
// sig = sigmoid(gate), writes the gradient that enters the attention, bf16(d_o * sig), to do_att
// (contiguous [B*S][N][H][Dt], what the main kernels read as their dO) and the gate's gradient
// d_o * O * sig * (1 - sig) to d_gate, and takes delta from the rounded do_att.
template <int DH>
__global__ void bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ o_resid,
                                const __nv_bfloat16* __restrict__ d_o, const float* __restrict__ lse,
                                const __nv_bfloat16* __restrict__ mask, uint4* __restrict__ xq,
                                uint4* __restrict__ xk, float inv_scale, int BS, int N, int H,
                                int NTP, ActLayout lay, int Dt, const __nv_bfloat16* __restrict__ gate,
                                __nv_bfloat16* __restrict__ do_att, __nv_bfloat16* __restrict__ d_gate) {
    constexpr uint32_t ONES = 0x3f803f80u;     // bf16 (1, 1)
    const size_t rows = static_cast<size_t>(BS) * N * H;
    const size_t gstride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const size_t t0 = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (size_t idx = t0; idx < rows; idx += gstride) {
        const int h = static_cast<int>(idx % H);
        const size_t bn = idx / H;
        const int n = static_cast<int>(bn % N);
        const size_t bs = bn / N;
        const size_t off = bs * lay.row + static_cast<size_t>(n) * lay.n + static_cast<size_t>(h) * lay.h;
        const uint4* po = reinterpret_cast<const uint4*>(o + off);
        const uint4* pr = o_resid ? reinterpret_cast<const uint4*>(o_resid + off) : nullptr;
        const uint4* pd = reinterpret_cast<const uint4*>(d_o + off);
        const uint4* pg = gate ? reinterpret_cast<const uint4*>(gate + off) : nullptr;
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < DH / 8; ++c) {
            if (c * 8 >= Dt) break;
            const uint4 a = po[c];
            uint4 b = pd[c];
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
            uint32_t rw[4] = {0u, 0u, 0u, 0u};
            if (pr) {
                const uint4 rr = pr[c];
                rw[0] = rr.x; rw[1] = rr.y; rw[2] = rr.z; rw[3] = rr.w;
            }
            if (pg) {
                const uint4 g4 = pg[c];
                const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, dw[4] = {b.x, b.y, b.z, b.w};
                uint32_t aw2[4], gg[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float s0 = 1.0f / (1.0f + ex2(-bf16_lo(gw[e]) * LOG2E));
                    const float s1 = 1.0f / (1.0f + ex2(-bf16_hi(gw[e]) * LOG2E));
                    const float d0 = bf16_lo(dw[e]), d1 = bf16_hi(dw[e]);
                    const float o0 = bf16_lo(aw[e]) + bf16_lo(rw[e]), o1 = bf16_hi(aw[e]) + bf16_hi(rw[e]);
                    aw2[e] = pack_bf16(d0 * s0, d1 * s1);
                    gg[e] = pack_bf16(d0 * o0 * s0 * (1.0f - s0), d1 * o1 * s1 * (1.0f - s1));
                }
                b = make_uint4(aw2[0], aw2[1], aw2[2], aw2[3]);
                reinterpret_cast<uint4*>(do_att + ((bs * N + n) * H + h) * static_cast<size_t>(Dt))[c] = b;
                reinterpret_cast<uint4*>(d_gate + off)[c] = make_uint4(gg[0], gg[1], gg[2], gg[3]);
            }
            const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s = fmaf(bf16_lo(aw[e]) + bf16_lo(rw[e]), bf16_lo(bw[e]), s);
                s = fmaf(bf16_hi(aw[e]) + bf16_hi(rw[e]), bf16_hi(bw[e]), s);
            }
        }
        const size_t ro = (bs * H + h) * NTP + n;
        xq[ro] = make_uint4(ONES, split_bf16(-lse[(bs * H + h) * N + n] * inv_scale), split_bf16(-s), 0u);
    }
    // padding of the per-row tiles, and the per-column tiles
    const int pad = NTP - N;
    const size_t npad = static_cast<size_t>(BS) * H * pad;
    for (size_t idx = t0; idx < npad; idx += gstride) {
        const size_t bh = idx / pad;
        const int n = N + static_cast<int>(idx % pad);
        xq[bh * NTP + n] = make_uint4(ONES, split_bf16(-1e30f), 0u, 0u);
    }
    const size_t nmask = static_cast<size_t>(BS) * NTP;
    for (size_t idx = t0; idx < nmask; idx += gstride) {
        const size_t bs = idx / NTP;
        const int n = static_cast<int>(idx % NTP);
        const float m = (n < N) ? __bfloat162float(mask[bs * N + n]) * inv_scale : -1e30f;
        xk[idx] = make_uint4(split_bf16(m), ONES, 0u, 0u);
    }
}

// fp32 accumulator [B*S][N][H][D] (contiguous) -> bf16 dQ in the activation layout, 8 elements per thread
template <int DH>
__global__ void cvt_dq_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n8, int N, int H,
                              ActLayout lay, int Dt) {
    const size_t gstride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += gstride) {
        const float4 a = reinterpret_cast<const float4*>(src)[2 * i];
        const float4 b = reinterpret_cast<const float4*>(src)[2 * i + 1];
        uint4 u;
        u.x = pack_bf16(a.x, a.y); u.y = pack_bf16(a.z, a.w);
        u.z = pack_bf16(b.x, b.y); u.w = pack_bf16(b.z, b.w);
        const size_t rowi = i / (DH / 8);                 // (bs, n, h) of this group of eight
        const int d8 = static_cast<int>(i % (DH / 8));
        if (d8 * 8 >= Dt) continue;
        const int h = static_cast<int>(rowi % H);
        const size_t bn = rowi / H;
        const size_t off = (bn / N) * lay.row + (bn % N) * lay.n + static_cast<size_t>(h) * lay.h + d8 * 8;
        *reinterpret_cast<uint4*>(dst + off) = u;
    }
}

struct BwdWorkspace {
    size_t off_xq, off_xk, off_dq, off_do, total;
};

static BwdWorkspace bwd_workspace(const EvoDims* d, bool gated = false) {
    const size_t BS = static_cast<size_t>(d->B) * d->S;
    const size_t NTP = static_cast<size_t>((d->N + TILE - 1) / TILE) * TILE;
    auto up = [](size_t x) { return (x + 255) & ~static_cast<size_t>(255); };
    BwdWorkspace w;
    w.off_xq = 0;
    w.off_xk = up(w.off_xq + BS * d->H * NTP * 16);
    w.off_dq = up(w.off_xk + BS * NTP * 16);
    const size_t dh = d->D <= 32 ? 32 : (d->D <= 64 ? 64 : 128);
    w.off_do = up(w.off_dq + BS * d->N * d->H * dh * 4);                         // fp32 dQ accumulator, kernel width
    w.total = gated ? up(w.off_do + BS * d->N * d->H * d->D * 2) : w.off_do;     // bf16 d_out * sigmoid(gate)
    return w;
}

template <int DH>
// lay_in: q, k, v; lay_out: o, o_resid, d_o, gate, d_gate; lay_grad: dq, dk, dv
static int launch_bwd(const EvoDims* d, const ActLayout& lay_in, const ActLayout& lay_out, const ActLayout& lay_grad,
                      const void* q, const void* k, const void* v, const void* bias,
                      const void* mask, const void* o, const void* o_resid, const float* lse, const void* d_o_in,
                      void* dq, void* dk, void* dv, float* dbias, uint8_t* ws, float scale, unsigned phases,
                      int reserved_sms, cudaStream_t st, const void* gate = nullptr, void* d_gate = nullptr) {
    using C = BwdCfg<DH>;
    const int BS = d->B * d->S;
    const int NT = (d->N + TILE - 1) / TILE;
    const BwdWorkspace w = bwd_workspace(d, gate != nullptr);
    // with a gate the kernels read the gradient entering the attention from the workspace (contiguous)
    const void* d_o = gate ? static_cast<const void*>(ws + w.off_do) : d_o_in;
    const ActLayout lay_do = gate ? contiguous_layout(d->N, d->H, d->D) : lay_out;
    uint4* xq = reinterpret_cast<uint4*>(ws + w.off_xq);
    uint4* xk = reinterpret_cast<uint4*>(ws + w.off_xk);
    float* dq_acc = reinterpret_cast<float*>(ws + w.off_dq);

    CUtensorMap tq, tk, tv, tdo, tb, tdq;
    int rc;
    const int Dt = d->D;          // 16 on the D = 32 kernel: boxes of 32 columns over tensors of 16
    if ((rc = make_tmap_qkv(&tq, q, BS, d->N, d->H, Dt, TILE, lay_in, RowTile<DH>::BOX_D))) return rc;
    if ((rc = make_tmap_qkv(&tk, k, BS, d->N, d->H, Dt, TILE, lay_in, RowTile<DH>::BOX_D))) return rc;
    if ((rc = make_tmap_qkv(&tv, v, BS, d->N, d->H, Dt, TILE, lay_in, RowTile<DH>::BOX_D))) return rc;
    if ((rc = make_tmap_qkv(&tdo, d_o, BS, d->N, d->H, Dt, TILE, lay_do, RowTile<DH>::BOX_D))) return rc;
    if ((rc = make_tmap_bias(&tb, bias, d->B, d->H, d->N))) return rc;
    if ((rc = make_tmap_rows_box(&tdq, dq_acc, 4, BS, d->N, d->H, DH, 32, 32))) return rc;

    BwdParams p;
    p.B = d->B; p.S = d->S; p.N = d->N; p.H = d->H;
    p.NT = NT;
    p.NTP = NT * TILE;
    p.CPB = (d->S + C::RC - 1) / C::RC;
    p.total_items = d->B * p.CPB * d->H * NT;
    p.scale = (scale > 0.f) ? scale : 1.0f / sqrtf(static_cast<float>(Dt));
    p.Dt = Dt;
    p.KB = (Dt + 15) / 16;
    p.c1 = p.scale * LOG2E;
    p.xq = reinterpret_cast<const __nv_bfloat16*>(xq);
    p.xk = reinterpret_cast<const __nv_bfloat16*>(xk);
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.dk = static_cast<__nv_bfloat16*>(dk); p.dv = static_cast<__nv_bfloat16*>(dv);
    p.lay = lay_grad;          // the kernel's own stores are dK and dV
    p.status = status_word();
    if (!p.status) return EVO_ERR_CUDA;

    int sms = 0;
    if ((rc = sm_count(&sms))) return rc;

    const size_t dq_bytes = static_cast<size_t>(BS) * d->N * d->H * DH * 4;
    const size_t db_bytes = static_cast<size_t>(d->B) * d->H * d->N * d->N * 4;

    // one S row and the whole backward in this call: the dQ/dK/dV kernel writes dBias (= dS) itself
    const bool dbias_here = (d->S == 1) && (phases & EVO_BWD_PHASE_DBIAS) && (phases & EVO_BWD_PHASE_DQKV);
    p.dbias = dbias;
    if (phases & EVO_BWD_PHASE_DBIAS) {
        if (!dbias_here && (rc = cuda_err(cudaMemsetAsync(dbias, 0, db_bytes, st)))) return rc;
        bwd_prep_kernel<DH><<<sms * 8, 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(o_resid),
            static_cast<const __nv_bfloat16*>(d_o_in), lse, static_cast<const __nv_bfloat16*>(mask), xq, xk,
            1.0f / p.scale, BS, d->N, d->H, p.NTP, lay_out, Dt, static_cast<const __nv_bfloat16*>(gate),
            reinterpret_cast<__nv_bfloat16*>(ws + w.off_do), static_cast<__nv_bfloat16*>(d_gate));
        if ((rc = cuda_err(cudaGetLastError()))) return rc;
        if (!dbias_here && (rc = launch_dbias(d, lay_in, lay_do, q, k, v, bias, d_o, xq, xk, dbias, scale, sms, st)))
            return rc;
    }
    if (!(phases & EVO_BWD_PHASE_DQKV)) return EVO_OK;

    if ((rc = cuda_err(cudaMemsetAsync(dq_acc, 0, dq_bytes, st)))) return rc;
    auto kernel = dbias_here ? evo_bwd_kernel<DH, true> : evo_bwd_kernel<DH, false>;
    if ((rc = set_max_smem_once(reinterpret_cast<const void*>(kernel), static_cast<int>(C::SMEM_BYTES))))
        return rc;
    // SMs left to other work (a collective on another stream) while this kernel runs
    int use_sms = sms - (reserved_sms > 0 ? reserved_sms : 0);
    if (use_sms < 1) use_sms = 1;
    const int grid = p.total_items < use_sms ? p.total_items : use_sms;
    prof_begin(1, st);
    kernel<<<grid, BWD_THREADS, C::SMEM_BYTES, st>>>(tq, tk, tv, tdo, tb, tdq, p);
    prof_end(1, st);
    if ((rc = cuda_err(cudaGetLastError()))) return rc;

    cvt_dq_kernel<DH><<<sms * 8, 256, 0, st>>>(dq_acc, static_cast<__nv_bfloat16*>(dq), dq_bytes / 32, d->N, d->H, lay_grad, Dt);
    return cuda_err(cudaGetLastError());
}

}  // namespace evo

// ---------------------------------------------------------------------------
// Backward with built-in scratch.  The workspace lives in a file-scope device
// array, so the call allocates nothing.  In host code the array's name is only a
// handle; its device address comes from cudaGetSymbolAddress, looked up once per
// device (with that device current) and kept.
// ---------------------------------------------------------------------------
#ifndef EVO_STATIC_SCRATCH_BYTES
#define EVO_STATIC_SCRATCH_BYTES (32u << 20)
#endif
static __device__ __align__(256) unsigned char g_bwd_scratch[EVO_STATIC_SCRATCH_BYTES];

namespace evo {
static int static_scratch(uint8_t** out) {
    static std::mutex mu;
    static uint8_t* cache[64] = {nullptr};
    int dev = 0;
    int rc = cuda_err(cudaGetDevice(&dev));
    if (rc) return rc;
    if (dev < 0 || dev >= 64) return EVO_ERR_CUDA;
    std::lock_guard<std::mutex> lock(mu);
    if (!cache[dev]) {
        void* ptr = nullptr;
        rc = cuda_err(cudaGetSymbolAddress(&ptr, g_bwd_scratch));
        if (rc) return rc;
        cache[dev] = static_cast<uint8_t*>(ptr);
    }
    *out = cache[dev];
    return EVO_OK;
}
}  // namespace evo

extern "C" size_t evo_bwd_static_scratch_capacity(void) { return EVO_STATIC_SCRATCH_BYTES; }

extern "C" int evo_bwd_static_scratch(const EvoDims* dims, const void* q, const void* k, const void* v,
                                      const void* pair_bias, const void* res_mask, const void* o,
                                      const void* o_resid, const float* lse, const void* d_o, void* dq, void* dk,
                                      void* dv, float* dbias, float scale, void* stream) {
    int rc = evo::check_dims(dims);
    if (rc) return rc;
    if (evo::bwd_workspace(dims).total > EVO_STATIC_SCRATCH_BYTES) return EVO_ERR_TOO_LARGE;
    if ((rc = evo::ensure_context())) return rc;
    uint8_t* scratch = nullptr;
    if ((rc = evo::static_scratch(&scratch))) return rc;
    return evo_bwd(dims, q, k, v, pair_bias, res_mask, o, o_resid, lse, d_o, dq, dk, dv, dbias, scratch,
                   EVO_STATIC_SCRATCH_BYTES, scale, stream);
}

extern "C" size_t evo_bwd_workspace_bytes(const EvoDims* dims) {
    if (evo::check_dims(dims) != EVO_OK) return 0;
    return evo::bwd_workspace(dims).total;
}

extern "C" int evo_bwd(const EvoDims* dims, const void* q, const void* k, const void* v,
                       const void* pair_bias, const void* res_mask, const void* o, const void* o_resid,
                       const float* lse, const void* d_o, void* dq, void* dk, void* dv, float* dbias,
                       void* workspace, size_t workspace_bytes, float scale, void* stream) {
    return evo_bwd_phased(dims, nullptr, q, k, v, pair_bias, res_mask, o, o_resid, lse, d_o, dq, dk, dv, dbias,
                          workspace, workspace_bytes, scale, EVO_BWD_PHASE_DBIAS | EVO_BWD_PHASE_DQKV, 0, stream);
}

extern "C" int evo_bwd_strided(const EvoDims* dims, const EvoStrides* strides, const void* q, const void* k,
                               const void* v, const void* pair_bias, const void* res_mask, const void* o,
                               const void* o_resid, const float* lse, const void* d_o, void* dq, void* dk,
                               void* dv, float* dbias, void* workspace, size_t workspace_bytes, float scale,
                               void* stream) {
    return evo_bwd_phased(dims, strides, q, k, v, pair_bias, res_mask, o, o_resid, lse, d_o, dq, dk, dv, dbias,
                          workspace, workspace_bytes, scale, EVO_BWD_PHASE_DBIAS | EVO_BWD_PHASE_DQKV, 0, stream);
}

extern "C" int evo_bwd_phased(const EvoDims* dims, const EvoStrides* strides, const void* q, const void* k,
                              const void* v, const void* pair_bias, const void* res_mask, const void* o,
                              const void* o_resid, const float* lse, const void* d_o, void* dq, void* dk,
                              void* dv, float* dbias, void* workspace, size_t workspace_bytes, float scale,
                              unsigned phases, int reserved_sms, void* stream) {
    return evo_bwd_gated(dims, strides, q, k, v, pair_bias, res_mask, nullptr, o, o_resid, lse, d_o, dq, dk, dv, nullptr,
                         dbias, workspace, workspace_bytes, scale, phases, reserved_sms, stream);
}

extern "C" size_t evo_bwd_gated_workspace_bytes(const EvoDims* dims) {
    if (evo::check_dims(dims) != EVO_OK) return 0;
    return evo::bwd_workspace(dims, true).total;
}

extern "C" int evo_bwd_gated(const EvoDims* dims, const EvoStrides* strides, const void* q, const void* k,
                             const void* v, const void* pair_bias, const void* res_mask, const void* gate,
                             const void* o, const void* o_resid, const float* lse, const void* d_o, void* dq,
                             void* dk, void* dv, void* d_gate, float* dbias, void* workspace,
                             size_t workspace_bytes, float scale, unsigned phases, int reserved_sms,
                             void* stream) {
    return evo_bwd_views(dims, strides, strides, strides, q, k, v, pair_bias, res_mask, gate, o, o_resid, lse, d_o, dq,
                         dk, dv, d_gate, dbias, workspace, workspace_bytes, scale, phases, reserved_sms, stream);
}

extern "C" int evo_bwd_views(const EvoDims* dims, const EvoStrides* s_qkv, const EvoStrides* s_out,
                             const EvoStrides* s_grad, const void* q, const void* k, const void* v,
                             const void* pair_bias, const void* res_mask, const void* gate, const void* o,
                             const void* o_resid, const float* lse, const void* d_o, void* dq, void* dk, void* dv,
                             void* d_gate, float* dbias, void* workspace, size_t workspace_bytes, float scale,
                             unsigned phases, int reserved_sms, void* stream) {
    int rc = evo::check_dims(dims);
    if (rc) return rc;
    if (!(phases & (EVO_BWD_PHASE_DBIAS | EVO_BWD_PHASE_DQKV))) return EVO_ERR_BAD_DIMS;
    evo::ActLayout lay, lay_out, lay_grad;
    if ((rc = evo::layout_from_strides(dims, s_qkv, &lay))) return rc;
    if ((rc = evo::layout_from_strides(dims, s_out, &lay_out))) return rc;
    if ((rc = evo::layout_from_strides(dims, s_grad, &lay_grad))) return rc;
    if (!q || !k || !v || !pair_bias || !res_mask || !o || !lse || !d_o || !dq || !dk || !dv || !dbias ||
        !workspace)
        return EVO_ERR_NULL_PTR;
    if ((gate == nullptr) != (d_gate == nullptr)) return EVO_ERR_NULL_PTR;
    const uintptr_t all = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                          reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(pair_bias) |
                          reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(d_o) |
                          reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) |
                          reinterpret_cast<uintptr_t>(dv) | reinterpret_cast<uintptr_t>(dbias) |
                          reinterpret_cast<uintptr_t>(lse) | reinterpret_cast<uintptr_t>(o_resid) |
                          reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(d_gate);
    if (all & 15u) return EVO_ERR_ALIGNMENT;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) ||
        workspace_bytes < evo::bwd_workspace(dims, gate != nullptr).total)
        return EVO_ERR_WORKSPACE;
    if ((rc = evo::ensure_context())) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    if (dims->D <= 32)
        return evo::launch_bwd<32>(dims, lay, lay_out, lay_grad, q, k, v, pair_bias, res_mask, o, o_resid, lse, d_o, dq, dk, dv, dbias,
                                   ws, scale, phases, reserved_sms, st, gate, d_gate);
    if (dims->D <= 64)
        return evo::launch_bwd<64>(dims, lay, lay_out, lay_grad, q, k, v, pair_bias, res_mask, o, o_resid, lse, d_o, dq, dk, dv, dbias,
                                   ws, scale, phases, reserved_sms, st, gate, d_gate);
    return evo::launch_bwd<128>(dims, lay, lay_out, lay_grad, q, k, v, pair_bias, res_mask, o, o_resid, lse, d_o, dq, dk, dv, dbias, ws,
                                scale, phases, reserved_sms, st, gate, d_gate);
}
