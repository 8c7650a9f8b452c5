// Launcher of the pair-bias gradient kernel (evo_dbias.cu), called by the
// backward launcher between its prep kernel and the dQ/dK/dV kernel.
#pragma once
#include "evo_host.cuh"

namespace evo {

// dbias [B][H][N][N] fp32 must be zeroed on `st` before the call.  xq and xk are the
// extra tiles the prep kernel writes (see evo_bwd.cu): bf16 [B*S][H][NTP][8] with the
// per-row terms and bf16 [B*S][NTP][8] with the per-column terms.
// `lay` gives the strides of q, k, v, `lay_do` those of d_o.
int launch_dbias(const EvoDims* d, const ActLayout& lay, const ActLayout& lay_do, const void* q, const void* k, const void* v, const void* bias,
                 const void* d_o, const void* xq, const void* xk, float* dbias, float scale, int sms, cudaStream_t st);

}  // namespace evo
