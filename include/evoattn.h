/* libevoattn -- EvoAttention (pair-bias + residue-mask attention) forward and
 * backward for NVIDIA B200 (sm_100a).  Plain C ABI: device pointers, sizes and
 * a CUDA stream; no framework types.  All tensors are caller-owned, contiguous
 * and 16-byte aligned.  Every call is asynchronous on `stream` and returns 0
 * (EVO_OK) or a negative error code; nothing throws, blocks or exits.
 *
 * Shapes (B batch, S MSA/triangle rows, N residues, H heads, D head dim):
 *   q,k,v,o,d_o,dq,dk,dv  bf16 [B][S][N][H][D]     (the caller layout of
 *                         evo_h100/tk_evo_attention_layer.py:5-11 -- no
 *                         transpose, no padding of D)
 *   pair_bias             bf16 [B][H][N][N]        (layer.py:91)
 *   res_mask              bf16 [B][S][N] additive  (layer.py:94)
 *   lse                   fp32 [B][S][H][N]  natural-log log-sum-exp
 *                         (evo_h100/tk_evoattention.cu:330-334)
 *   dbias                 fp32 [B][H][N][N]        (tk_evoattention.cu:1113)
 * Supported: D in {16, 32, 64, 96, 128}, the head dims of the reference's kernels
 * and test grids (evo_h100/test_tk_evoattention.py:89-103).  16 runs on the D = 32
 * kernels and 96 on the D = 128 kernels: their loads zero-fill and their stores clip
 * the missing columns, no padded copy is made;
 * N a multiple of 8 (any N >= 8, the last tile may be ragged);
 * N*H*D*S*B*2 bytes < 2^40.
 */
#ifndef EVOATTN_H_
#define EVOATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct EvoDims {
    int32_t B, S, N, H, D;
} EvoDims;

/* Element strides of the five-dimensional activation tensors (q, k, v, o, o_resid,
 * d_o, dq, dk, dv) along B, N_SEQ, N_CTX and H; the head dimension is always
 * contiguous.  The contiguous layout of the reference's callers
 * (evo_h100/tk_evo_attention_layer.py:5-11) is {S*N*H*D, N*H*D, H*D, D}.  Every
 * stride must be a multiple of 8 elements (16 bytes), and either B == 1 or
 * b == S * s, so that (B, N_SEQ) flatten into one axis. */
typedef struct EvoStrides {
    int64_t b, s, n, h;
} EvoStrides;

enum {
    EVO_OK = 0,
    EVO_ERR_BAD_DIMS = -1,      /* unsupported D / N / non-positive extent        */
    EVO_ERR_NULL_PTR = -2,
    EVO_ERR_ALIGNMENT = -3,     /* a pointer is not 16-byte aligned               */
    EVO_ERR_WORKSPACE = -4,     /* workspace smaller than evo_bwd_workspace_bytes */
    EVO_ERR_NO_DRIVER = -5,     /* CUDA driver / tensor-map encoder unavailable   */
    EVO_ERR_TENSOR_MAP = -6,    /* cuTensorMapEncodeTiled refused the layout      */
    EVO_ERR_CUDA = -7,          /* a CUDA runtime call failed (see evo_last_cuda_error) */
    EVO_ERR_DEVICE_WAIT = -8,   /* a kernel's bounded wait ran out (evo_device_status) */
    EVO_ERR_TOO_LARGE = -9      /* problem exceeds a fixed-capacity entry point   */
};

/* Library ABI version (major*100 + minor). */
int evo_version(void);
const char* evo_strerror(int code);
/* cudaError_t of the most recent failing runtime call on this thread (0 if none). */
int evo_last_cuda_error(void);
/* Text describing the most recent tensor-map encoding failure on this thread ("" if none). */
const char* evo_last_error_detail(void);

/* Forward.  Replaces evoattention_forward (evo_h100/tk_evoattention.cu:911-1043):
 * O = softmax(q k^T * scale + pair_bias + res_mask) v, LSE saved for backward.
 * scale <= 0 means 1/sqrt(D) (tk_evoattention.cu:988-990).  Unlike the
 * reference it does not allocate outputs and does not synchronise the stream
 * (tk_evoattention.cu:977-978, :1040).
 * o_resid (optional, may be NULL): bf16 [B][S][N][H][D] that receives the
 * rounding residual O_fp32 - bf16(O).  Passing it on to evo_bwd makes
 * delta = rowsum(dO o O) accurate to about 16 bits of O instead of 8, which
 * keeps the error of dBias (a sum over S rows) within 2e-2 at large S. */
int evo_fwd(const EvoDims* dims, const void* q, const void* k, const void* v,
            const void* pair_bias, const void* res_mask, void* o, void* o_resid, float* lse,
            float scale, void* stream);

/* evo_fwd / evo_bwd for activation tensors that are views with the strides given
 * (all nine tensors share them): what the reference's callers get by transposing
 * and copying (evo_h100/tk_evo_attention_layer.py:81-102,146-173) -- for instance the
 * "ending node" triangle attention, whose N_SEQ and N_CTX axes are swapped in memory --
 * is read and written in place through the tensor maps.  pair_bias, res_mask, lse,
 * dbias and the workspace are contiguous as in evo_fwd / evo_bwd.  strides == NULL
 * means the contiguous layout.  EVO_ERR_BAD_DIMS for strides that break the rules
 * given at EvoStrides. */
int evo_fwd_strided(const EvoDims* dims, const EvoStrides* strides, const void* q, const void* k,
                    const void* v, const void* pair_bias, const void* res_mask, void* o, void* o_resid,
                    float* lse, float scale, void* stream);
int evo_bwd_strided(const EvoDims* dims, const EvoStrides* strides, const void* q, const void* k,
                    const void* v, const void* pair_bias, const void* res_mask, const void* o,
                    const void* o_resid, const float* lse, const void* d_o, void* dq, void* dk, void* dv,
                    float* dbias, void* workspace, size_t workspace_bytes, float scale, void* stream);

/* evo_bwd_strided in two separately launchable phases, for S-sharded multi-GPU
 * callers (no counterpart in the reference, which is single-GPU):
 *   EVO_BWD_PHASE_DBIAS  prep + the dBias kernel: dbias is complete when this phase is
 *   EVO_BWD_PHASE_DQKV   the dQ/dK/dV kernel and the dQ conversion; needs the rows the
 *                        first phase left in `workspace` (same workspace, same stream
 *                        order), and leaves `reserved_sms` SMs unused
 * so that the caller can start the all-reduce of dbias on another stream between the
 * two calls and have it run on the reserved SMs next to the second phase.  Both bits
 * and reserved_sms = 0 is evo_bwd_strided. */
enum { EVO_BWD_PHASE_DBIAS = 1, EVO_BWD_PHASE_DQKV = 2 };
int evo_bwd_phased(const EvoDims* dims, const EvoStrides* strides, const void* q, const void* k,
                   const void* v, const void* pair_bias, const void* res_mask, const void* o,
                   const void* o_resid, const float* lse, const void* d_o, void* dq, void* dk, void* dv,
                   float* dbias, void* workspace, size_t workspace_bytes, float scale, unsigned phases,
                   int reserved_sms, void* stream);

/* Bytes of scratch evo_bwd needs for these dims (per-row and per-column extra tiles of the
 * logits + fp32 dQ accumulator). */
size_t evo_bwd_workspace_bytes(const EvoDims* dims);

/* Backward.  Replaces evoattention_backward (tk_evoattention.cu:1051-1197):
 * recomputes P from LSE; dq = scale * dS k, dk = scale * dS^T q, dv = P^T d_o,
 * dbias = sum over S of dS (unscaled, tk_evoattention.cu:824-833), dS = P o (dP - delta).
 * dq/dk/dv are written as bf16 in the caller layout (the reference returns
 * padded fp32, tk_evoattention.cu:1109-1112); dbias (fp32) is overwritten, not
 * accumulated into.  o_resid is the optional residual written by evo_fwd (NULL:
 * delta is computed from the bf16 O alone).  `workspace` is scratch of at least
 * evo_bwd_workspace_bytes(dims), 256-byte aligned; its contents are undefined
 * afterwards. */
int evo_bwd(const EvoDims* dims, const void* q, const void* k, const void* v,
            const void* pair_bias, const void* res_mask, const void* o, const void* o_resid,
            const float* lse, const void* d_o, void* dq, void* dk, void* dv, float* dbias,
            void* workspace, size_t workspace_bytes, float scale, void* stream);

/* Backward for callers that may not allocate device memory -- no counterpart in
 * the reference.  Same computation and arguments as evo_bwd, minus the
 * workspace: the scratch is a fixed array inside the library
 * (evo_bwd_static_scratch_capacity() bytes, 32 MiB by default), so this call
 * makes no cudaMalloc / cudaFree and uses no allocating library routine.  It is
 * meant for hosts where device memory is handed out up front and nothing may
 * be allocated afterwards: an inference or training server whose memory pool
 * already owns the whole GPU, a plugin loaded into such a process, or code that
 * runs where an allocation would stall or fail (for example inside a section
 * the host has frozen against allocator calls).
 *   - Problems whose evo_bwd_workspace_bytes(dims) exceeds the capacity are
 *     refused with EVO_ERR_TOO_LARGE; nothing is launched.
 *   - The first call on each device looks up the array's device address (once,
 *     with that device current).  Make that first call before any stream
 *     capture begins on the device.
 *   - Every call on a device shares the one array and leaves its last contents
 *     there; the call itself re-zeroes the part that must start at zero.  Two
 *     calls that overlap on the same GPU (different streams, or different
 *     threads) race on the scratch: serialise them.
 *   - Every GPU that loads the library holds the array until the process exits. */
size_t evo_bwd_static_scratch_capacity(void);
int evo_bwd_static_scratch(const EvoDims* dims, const void* q, const void* k, const void* v,
                           const void* pair_bias, const void* res_mask, const void* o,
                           const void* o_resid, const float* lse, const void* d_o, void* dq, void* dk,
                           void* dv, float* dbias, float scale, void* stream);

/* Forward and backward with the sigmoid gate that follows this attention in the
 * AlphaFold-3 / MegaFold blocks fused in: out = sigmoid(gate) * O.  The reference has
 * no such entry point (its callers multiply in a separate elementwise pass,
 * evo_h100/README.md:655-669 discusses the cost of the passes around the kernel);
 * the arguments it shares with evo_fwd_strided / evo_bwd_phased mean the same.
 *   gate     bf16, the layout of q: the gate's pre-activation logits
 *   o        still receives the un-gated attention output: backward needs it
 *   o_gated  bf16, the layout of q: sigmoid(gate) * O, formed from the unrounded O
 * gate == NULL and o_gated == NULL together make this evo_fwd_strided. */
int evo_fwd_gated(const EvoDims* dims, const EvoStrides* strides, const void* q, const void* k,
                  const void* v, const void* pair_bias, const void* res_mask, const void* gate,
                  void* o, void* o_gated, void* o_resid, float* lse, float scale, void* stream);
/*   d_out    gradient of the loss with respect to o_gated (bf16, the layout of q)
 *   d_gate   receives the gradient with respect to the gate logits (bf16, the layout of q):
 *            d_out * O * sigmoid(gate) * (1 - sigmoid(gate))
 * The gradient that flows into the attention, d_out * sigmoid(gate), is formed by the
 * prep kernel into the workspace (evo_bwd_gated_workspace_bytes, larger than
 * evo_bwd_workspace_bytes by one bf16 activation tensor). */
size_t evo_bwd_gated_workspace_bytes(const EvoDims* dims);
int evo_bwd_gated(const EvoDims* dims, const EvoStrides* strides, const void* q, const void* k,
                  const void* v, const void* pair_bias, const void* res_mask, const void* gate,
                  const void* o, const void* o_resid, const float* lse, const void* d_out, void* dq,
                  void* dk, void* dv, void* d_gate, float* dbias, void* workspace, size_t workspace_bytes,
                  float scale, unsigned phases, int reserved_sms, void* stream);

/* The same two calls with separate views for the three families of activation tensors
 * (no counterpart in the reference, whose wrapper copies every tensor into one layout,
 * evo_h100/tk_evo_attention_layer.py:81-102):
 *   s_qkv   q, k, v                                   (read)
 *   s_out   o, o_resid, o_gated, gate, d_out, d_gate  (the output side)
 *   s_grad  dq, dk, dv                                (written by the backward)
 * Each is an EvoStrides as in evo_fwd_strided, or NULL for contiguous.  A view need not be
 * dense: q, k and v sliced out of one fused projection [B][S][N][3][H][D] are read where
 * they lie, while O and the gradients are written contiguously. */
int evo_fwd_views(const EvoDims* dims, const EvoStrides* s_qkv, const EvoStrides* s_out, const void* q,
                  const void* k, const void* v, const void* pair_bias, const void* res_mask,
                  const void* gate, void* o, void* o_gated, void* o_resid, float* lse, float scale,
                  void* stream);
int evo_bwd_views(const EvoDims* dims, const EvoStrides* s_qkv, const EvoStrides* s_out,
                  const EvoStrides* s_grad, const void* q, const void* k, const void* v,
                  const void* pair_bias, const void* res_mask, const void* gate, const void* o,
                  const void* o_resid, const float* lse, const void* d_out, void* dq, void* dk, void* dv,
                  void* d_gate, float* dbias, void* workspace, size_t workspace_bytes, float scale,
                  unsigned phases, int reserved_sms, void* stream);

/* Reads (and clears) the device status word that kernels set when a bounded
 * wait gives up.  Synchronises the device.  Returns EVO_OK, EVO_ERR_DEVICE_WAIT
 * (raw word in *raw if non-NULL) or EVO_ERR_CUDA.  The reference has no
 * counterpart: its kernels wait without bound. */
int evo_device_status(uint32_t* raw);

/* Optional timing of the three main kernels with CUDA events recorded on the
 * caller's stream around each launch (no counterpart in the reference, which
 * times whole calls from Python, evo_h100/benchmark.py:76-124).
 * evo_profile_enable(1) starts recording (at most 4096 launches per kernel are
 * kept), evo_profile_enable(0) stops.  evo_profile_read waits for the recorded
 * events, returns the summed milliseconds and the launch count of
 * kernel 0 (forward), 1 (backward dQ/dK/dV kernel) or 2 (backward dBias kernel),
 * and clears that record. */
int evo_profile_enable(int on);
int evo_profile_read(int kernel, float* total_ms, int* launches);

/* Unit check of the tensor-core operand conventions used by the kernels (no
 * counterpart in the reference).  x: bf16 [128][128], y, z: bf16 [128][D].
 *   out_yzt [128][128] = y z^T      (both operands K-major row tiles)
 *   out_xy  [128][D]   = x y        (A K-major square tile, B MN-major row tile)
 *   out_xty [128][D]   = x^T y      (A MN-major square tile, B MN-major row tile)
 *   out_ts  [128][D]   = x y        (A in tensor memory, B MN-major row tile)
 * all fp32. */
int evo_selftest_mma(int D, const void* x, const void* y, const void* z, float* out_yzt,
                     float* out_xy, float* out_xty, float* out_ts, void* stream);

/* Unit check of the extra contraction block the backward kernels append to their
 * logit products (no counterpart in the reference): y, z bf16 [128][D]; a, b bf16
 * [128][8], 16-byte aligned; out fp32 [128][128] = y z^T + a b^T. */
int evo_selftest_mma_extra(int D, const void* y, const void* z, const void* a, const void* b,
                           float* out, void* stream);

/* Exercises the give-up path of the kernels' bounded waits without any fault (no
 * counterpart in the reference, whose kernels wait without bound): one CTA waits on
 * a barrier that nothing arrives at, with a limit of `limit_ns` nanoseconds
 * (1 .. 100,000,000), records the time-out in the device status word, releases its
 * other warp through the CTA's abort flag (*released, a device word, becomes 1) and
 * returns normally.  evo_device_status afterwards reports EVO_ERR_DEVICE_WAIT with
 * raw = (1 << 16) | 0xee, and clears the word. */
int evo_selftest_wait_timeout(unsigned long long limit_ns, unsigned int* released, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* EVOATTN_H_ */
