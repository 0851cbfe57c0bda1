// Gated linear attention: the per-head matrix state S [D x Dv] with one decay per key channel,
//     S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,     o_t = S_t^T q_t,
// advanced token by token in fp32, for prompts (S tokens per row) and for decoding (S = 1) alike.
//
// The decay comes from a low-rank projection: z = A2 (A1 h) + bias, alpha = sigmoid(z)^(1/tau) = exp(logsigmoid(z) / tau).
// The rank-R product A1 h arrives as R fp32 columns of the fused projection buffer; the A2 product, the bias, the
// log-sigmoid and the exponential are done here in fp32 for a chunk of tokens at a time.
//
// Work split: grid (value-column slices, heads, batch rows); a thread owns GS_DP = 32 key channels of one value column of
// the state in registers, P = ceil(D / 32) (rounded to a power of two) adjacent lanes share a column and add their
// partial o with shuffles.  q, k and alpha of a chunk of tokens are staged in shared memory, one row of 33 floats per
// 32 channels so that the P lanes of a column read different banks.  Padding tokens (slot < pad_left[b]) are skipped:
// the state of a left-padded row starts at its first real token.
#include "jllama_b200.h"
#include "seq_types.cuh"

namespace jl {

constexpr int GS_DP = 32;        // state rows per thread
constexpr int GS_TC = 8;         // tokens staged per chunk
constexpr int GS_THREADS = 128;

struct GlaParams {
  const float* y; int ldy;
  int q_off, k_off, v_off, a_off;      // columns of y: q [H*D], k [H*D], v [H*Dv], low-rank decay input [R]
  int B, S, H, D, Dv, R, P;
  float q_scale, inv_tau;
  const int* cache_len; const int* pad_left;
  float* state;                        // [B][H][D][Dv] fp32, read and written
  float* o;                            // [B*S][H][Dv] fp32
};

__device__ __forceinline__ float log_sigmoid(float z) {
  return z >= 0.0f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
}

template <typename T>
__global__ void __launch_bounds__(GS_THREADS) gla_scan_kernel(GlaParams p, const T* __restrict__ a2, const T* __restrict__ a2b) {
  extern __shared__ float smem[];
  const int P = p.P;                                         // lanes per value column (power of two, adjacent lanes of a warp)
  const int cols = GS_THREADS / P;                           // value columns per CTA
  const int tid = threadIdx.x;
  const int part = tid % P, lcol = tid / P, col = blockIdx.x * cols + lcol;
  const int h = blockIdx.y, b = blockIdx.z;
  const int DS = P * (GS_DP + 1);                            // padded channel pitch of one token's q / k / alpha
  float* qs = smem;                                          // [TC][DS]
  float* ks = qs + GS_TC * DS;
  float* as = ks + GS_TC * DS;
  float* vs = as + GS_TC * DS;                               // [TC][cols]
  float* zs = vs + GS_TC * cols;                             // [TC][R]

  float st[GS_DP];
  const int d0 = part * GS_DP;
  float* sbase = p.state + (((size_t)b * p.H + h) * p.D) * p.Dv;
#pragma unroll
  for (int r = 0; r < GS_DP; ++r) st[r] = (col < p.Dv && d0 + r < p.D) ? sbase[(size_t)(d0 + r) * p.Dv + col] : 0.0f;

  const int first = max(0, (p.pad_left ? p.pad_left[b] : 0) - (p.cache_len ? *p.cache_len : 0));   // first real token of this call
  if (part == 0 && col < p.Dv)                               // padding tokens: defined (zero) output rows
    for (int s = 0; s < min(first, p.S); ++s) p.o[((size_t)(b * p.S + s) * p.H + h) * p.Dv + col] = 0.0f;
  for (int s0 = first; s0 < p.S; s0 += GS_TC) {
    const int nt = min(GS_TC, p.S - s0);
    __syncthreads();
    for (int i = tid; i < nt * p.R; i += GS_THREADS) {
      const int t = i / p.R, r = i % p.R;
      zs[t * p.R + r] = p.y[(size_t)(b * p.S + s0 + t) * p.ldy + p.a_off + r];
    }
    for (int i = tid; i < nt * cols; i += GS_THREADS) {
      const int t = i / cols, c = blockIdx.x * cols + i % cols;
      vs[i] = c < p.Dv ? p.y[(size_t)(b * p.S + s0 + t) * p.ldy + p.v_off + h * p.Dv + c] : 0.0f;
    }
    __syncthreads();
    for (int i = tid; i < nt * P * GS_DP; i += GS_THREADS) {
      const int t = i / (P * GS_DP), d = i % (P * GS_DP);
      const int at = t * DS + (d / GS_DP) * (GS_DP + 1) + d % GS_DP;
      float qv = 0.0f, kv = 0.0f, av = 1.0f;
      if (d < p.D) {
        const float* yr = p.y + (size_t)(b * p.S + s0 + t) * p.ldy;
        qv = yr[p.q_off + h * p.D + d] * p.q_scale;
        kv = yr[p.k_off + h * p.D + d];
        const int n = h * p.D + d;
        float z = to_f(a2b[n]);
        for (int r = 0; r < p.R; ++r) z = fmaf(to_f(a2[(size_t)n * p.R + r]), zs[t * p.R + r], z);
        av = expf(log_sigmoid(z) * p.inv_tau);
      }
      qs[at] = qv; ks[at] = kv; as[at] = av;
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float v = vs[t * cols + lcol];
      const float* qt = qs + t * DS + part * (GS_DP + 1);
      const float* kt = ks + t * DS + part * (GS_DP + 1);
      const float* at = as + t * DS + part * (GS_DP + 1);
      float acc = 0.0f;
#pragma unroll
      for (int r = 0; r < GS_DP; ++r) {
        st[r] = fmaf(at[r], st[r], kt[r] * v);
        acc = fmaf(qt[r], st[r], acc);
      }
      for (int off = P >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (part == 0 && col < p.Dv) p.o[((size_t)(b * p.S + s0 + t) * p.H + h) * p.Dv + col] = acc;
    }
  }
#pragma unroll
  for (int r = 0; r < GS_DP; ++r)
    if (col < p.Dv && d0 + r < p.D) sbase[(size_t)(d0 + r) * p.Dv + col] = st[r];
}

}  // namespace jl

using namespace jl;

extern "C" JL_API int jl_gla_scan(const float* y, int ldy, int q_off, int k_off, int v_off, int a_off, const void* a2,
                                  const void* a2_bias, float* state, float* o, const int* cache_len, const int* pad_left, int B,
                                  int S, int H, int D, int Dv, int R, float q_scale, float tau, int dtype, void* stream) {
  JL_CHECK_ARG(B >= 1 && S >= 1 && H >= 1 && D >= 1 && Dv >= 1 && R >= 1, "jl_gla_scan: bad shape");
  JL_CHECK_ARG(tau > 0.0f, "jl_gla_scan: tau=%f must be positive", tau);
  int P = 1;
  while (P * GS_DP < D) P *= 2;
  JL_CHECK_ARG(P <= 32, "jl_gla_scan: key size %d above %d", D, 32 * GS_DP);
  const int cols = GS_THREADS / P;
  GlaParams p{y, ldy, q_off, k_off, v_off, a_off, B, S, H, D, Dv, R, P, q_scale, 1.0f / tau, cache_len, pad_left, state, o};
  const size_t smem = (size_t)(3 * GS_TC * P * (GS_DP + 1) + GS_TC * cols + GS_TC * R) * sizeof(float);
  JL_CHECK_ARG(smem <= 200 * 1024, "jl_gla_scan: key size %d with rank %d does not fit the staging buffer", D, R);
  dim3 grid((Dv + cols - 1) / cols, H, B), block(GS_THREADS);
  count_launch();
  if (smem > 48 * 1024) {
    if (dtype == DT_BF16) JL_CUDA(cudaFuncSetAttribute(gla_scan_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    else JL_CUDA(cudaFuncSetAttribute(gla_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  JL_DISPATCH_DTYPE(dtype, gla_scan_kernel<T><<<grid, block, smem, (cudaStream_t)stream>>>(p, (const T*)a2, (const T*)a2_bias));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}
