// Softmax attention for any head sizes (query/key size D, value size Dv, D != Dv allowed), grouped key/value heads, in
// bfloat16 or true float32, with the pieces newer decoder designs put around it:
//
//  * attn_prep_kernel   — interleaved-pair rotary embedding on the first `rot` channels of each head (pair 2i, 2i+1;
//    the rest pass through), then optional weight-free unit-RMS scaling of q and k per head, append of k / v to the
//    cache [B][G][T][D] / [B][G][T][Dv].  Token (b, s) goes to slot *cache_len + s at position slot - pad_left[b].
//    A layer that reads another layer's keys and values runs it for the queries only.
//  * attn_rows_kernel   — one warp per query: blocks of 32 keys (one key per lane for the scores, one value column per
//    lane for the output), online softmax in fp32, causal over slots [pad_left[b], slot], optional per-head output
//    gate sigmoid(g).  Prompts of any length; exact fall-back for head sizes the tensor-core kernels are not built for.
//  * attn_decode_kernel — one CTA per (row, head) for a single new token: its warps take interleaved blocks of 32 keys
//    and merge their (max, sum, output) triples in shared memory.
//
// Input q / k / v / gate are columns of one fp32 projection buffer (row pitch ldy), as the fused projection writes them.
#include "jllama_b200.h"
#include "seq_types.cuh"

namespace jl {

struct PrepParams {
  const float* y; int ldy;
  int q_off, k_off, v_off;          // column offsets in y; k_off < 0: queries only
  int B, S, H, G, D, Dv, T;
  int rot;                          // rotated channels per head (even, <= D)
  const float* cos_t; const float* sin_t; int max_pos;      // [max_pos][rot/2]
  int unit_norm; float eps;
  const int* cache_len; const int* pad_left;
};

constexpr int AP_WARPS = 4;      // heads per CTA of the preparation kernel (one warp each)

template <typename T>
__global__ void __launch_bounds__(AP_WARPS * 32) attn_prep_kernel(PrepParams p, T* __restrict__ q_out, T* __restrict__ kc,
                                                                  T* __restrict__ vc, int n_heads, int pair_loads) {
  const int m = blockIdx.x, head = blockIdx.y * AP_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (head >= n_heads) return;
  const int b = m / p.S, s = m % p.S;
  const int slot = (p.cache_len ? *p.cache_len : 0) + s;
  int pos = slot - (p.pad_left ? p.pad_left[b] : 0);
  pos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
  const float* yr = p.y + (size_t)m * p.ldy;
  if (head >= p.H + p.G) {                               // value head: plain copy into the cache
    const int g = head - p.H - p.G;
    T* dst = vc + (((size_t)b * p.G + g) * p.T + slot) * p.Dv;
    for (int i = lane; i < p.Dv; i += 32) dst[i] = from_f<T>(yr[p.v_off + g * p.Dv + i]);
    return;
  }
  const bool is_q = head < p.H;
  const float* src = yr + (is_q ? p.q_off + head * p.D : p.k_off + (head - p.H) * p.D);
  T* dst = is_q ? q_out + ((size_t)m * p.H + head) * p.D
                : kc + (((size_t)b * p.G + (head - p.H)) * p.T + slot) * p.D;
  const float* ct = p.cos_t + (size_t)pos * (p.rot / 2);
  const float* st = p.sin_t + (size_t)pos * (p.rot / 2);
  const int npairs = p.D / 2 + (p.D & 1);
  // pass 1 rotates and sums the squares, pass 2 rotates again (L1 hits) and writes the scaled values
  float r = 1.0f;
  for (int pass = p.unit_norm ? 0 : 1; pass < 2; ++pass) {
    float ss = 0.0f;
    for (int i = lane; i < npairs; i += 32) {
      const int c0 = 2 * i, c1 = 2 * i + 1;
      float u, v;
      if (pair_loads) { const float2 t = *reinterpret_cast<const float2*>(src + c0); u = t.x; v = t.y; }
      else { u = src[c0]; v = c1 < p.D ? src[c1] : 0.0f; }
      if (c1 < p.rot) { const float c = ct[i], sn = st[i]; const float ru = u * c - v * sn, rv = v * c + u * sn; u = ru; v = rv; }
      if (pass == 0) {
        ss += u * u + v * v;
      } else {
        dst[c0] = from_f<T>(u * r);
        if (c1 < p.D) dst[c1] = from_f<T>(v * r);
      }
    }
    if (pass == 0) r = 1.0f / sqrtf(warp_sum(ss) / (float)p.D + p.eps);
  }
}

struct AttnParams {
  int B, S, H, G, D, Dv, T;
  float scale;
  const int* cache_len;             // slots already filled BEFORE this call's tokens (device scalar); nullptr = 0
  const int* pad_left;
  const float* gate; int ldg;       // fp32 pre-activation of the per-head output gate (column h of row m), or nullptr
};

constexpr int AT_MAXV = 16;         // value columns per lane: Dv <= 512

// scores of one block of 32 keys (lane = key), then the block's contribution to the output (lane = value column)
template <typename T>
__device__ __forceinline__ void attn_block(const float* __restrict__ qs, const T* __restrict__ kbase, const T* __restrict__ vbase,
                                           int j0, int lo, int hi, int D, int Dv, float scale, float& mrun, float& lrun,
                                           float (&acc)[AT_MAXV]) {
  const int lane = threadIdx.x & 31;
  const int j = j0 + lane;
  float sc = -INFINITY;
  if (j >= lo && j <= hi) {
    const T* kr = kbase + (size_t)j * D;
    float d = 0.0f;
    for (int c = 0; c < D; ++c) d = fmaf(qs[c], to_f(kr[c]), d);
    sc = d * scale;
  }
  const float mnew = fmaxf(mrun, warp_max(sc));
  if (mnew == -INFINITY) return;                       // nothing visible in this block (uniform across the warp)
  const float corr = mrun == -INFINITY ? 0.0f : expf(mrun - mnew);
  const float pj = sc == -INFINITY ? 0.0f : expf(sc - mnew);
  lrun = lrun * corr + warp_sum(pj);
  mrun = mnew;
#pragma unroll
  for (int i = 0; i < AT_MAXV; ++i) acc[i] *= corr;
  const int jend = min(32, hi - j0 + 1);
  for (int t = 0; t < jend; ++t) {
    const float pt = __shfl_sync(0xffffffffu, pj, t);
    if (pt == 0.0f) continue;
    const T* vr = vbase + (size_t)(j0 + t) * Dv;
#pragma unroll
    for (int i = 0; i < AT_MAXV; ++i) {
      const int c = lane + 32 * i;
      if (c < Dv) acc[i] = fmaf(pt, to_f(vr[c]), acc[i]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) attn_rows_kernel(AttnParams p, const T* __restrict__ q, const T* __restrict__ kc,
                                                        const T* __restrict__ vc, T* __restrict__ out) {
  extern __shared__ float smem[];                       // [warps][D] queries in fp32
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int h = blockIdx.y, b = blockIdx.z;
  const int s = blockIdx.x * nw + warp;
  if (s >= p.S) return;
  const int m = b * p.S + s;
  const int g = h / (p.H / p.G);
  float* qs = smem + warp * p.D;
  const T* qr = q + ((size_t)m * p.H + h) * p.D;
  for (int c = lane; c < p.D; c += 32) qs[c] = to_f(qr[c]);
  __syncwarp();
  const int lo = p.pad_left ? p.pad_left[b] : 0;
  const int hi = (p.cache_len ? *p.cache_len : 0) + s;   // own slot: the last visible key
  const T* kbase = kc + ((size_t)b * p.G + g) * p.T * p.D;
  const T* vbase = vc + ((size_t)b * p.G + g) * p.T * p.Dv;
  float mrun = -INFINITY, lrun = 0.0f, acc[AT_MAXV] = {};
  for (int j0 = lo & ~31; j0 <= hi; j0 += 32) attn_block<T>(qs, kbase, vbase, j0, lo, hi, p.D, p.Dv, p.scale, mrun, lrun, acc);
  float gmul = lrun > 0.0f ? 1.0f / lrun : 0.0f;         // a padding query sees nothing: its row is zero
  if (p.gate) gmul *= sigmoid_f(p.gate[(size_t)m * p.ldg + h]);
#pragma unroll
  for (int i = 0; i < AT_MAXV; ++i) {
    const int c = lane + 32 * i;
    if (c < p.Dv) out[((size_t)m * p.H + h) * p.Dv + c] = from_f<T>(acc[i] * gmul);
  }
}

constexpr int AD_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(AD_WARPS * 32) attn_decode_kernel(AttnParams p, const T* __restrict__ q, const T* __restrict__ kc,
                                                                    const T* __restrict__ vc, T* __restrict__ out) {
  extern __shared__ float smem[];                       // [D] query | [warps][2] (max, sum) | [warps][Dv] partial outputs
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.y;             // S == 1: row m = b
  const int g = h / (p.H / p.G);
  float* qs = smem;
  float* ml = smem + p.D;
  float* part = ml + 2 * AD_WARPS;
  const T* qr = q + ((size_t)b * p.H + h) * p.D;
  for (int c = threadIdx.x; c < p.D; c += blockDim.x) qs[c] = to_f(qr[c]);
  __syncthreads();
  const int lo = p.pad_left ? p.pad_left[b] : 0;
  const int hi = p.cache_len ? *p.cache_len : 0;
  const T* kbase = kc + ((size_t)b * p.G + g) * p.T * p.D;
  const T* vbase = vc + ((size_t)b * p.G + g) * p.T * p.Dv;
  float mrun = -INFINITY, lrun = 0.0f, acc[AT_MAXV] = {};
  for (int j0 = (lo & ~31) + 32 * warp; j0 <= hi; j0 += 32 * AD_WARPS)
    attn_block<T>(qs, kbase, vbase, j0, lo, hi, p.D, p.Dv, p.scale, mrun, lrun, acc);
  if (lane == 0) { ml[2 * warp] = mrun; ml[2 * warp + 1] = lrun; }
#pragma unroll
  for (int i = 0; i < AT_MAXV; ++i) {
    const int c = lane + 32 * i;
    if (c < p.Dv) part[warp * p.Dv + c] = acc[i];
  }
  __syncthreads();
  float mall = -INFINITY;
  for (int w = 0; w < AD_WARPS; ++w) mall = fmaxf(mall, ml[2 * w]);
  float lall = 0.0f;
  for (int w = 0; w < AD_WARPS; ++w) if (ml[2 * w] != -INFINITY) lall += ml[2 * w + 1] * expf(ml[2 * w] - mall);
  float gmul = lall > 0.0f ? 1.0f / lall : 0.0f;
  if (p.gate) gmul *= sigmoid_f(p.gate[(size_t)b * p.ldg + h]);
  for (int c = threadIdx.x; c < p.Dv; c += blockDim.x) {
    float o = 0.0f;
    for (int w = 0; w < AD_WARPS; ++w) if (ml[2 * w] != -INFINITY) o += part[w * p.Dv + c] * expf(ml[2 * w] - mall);
    out[((size_t)b * p.H + h) * p.Dv + c] = from_f<T>(o * gmul);
  }
}

// out[m, h, :] *= sigmoid(gate[m, h]) for attention kernels that have no gate input (the tcgen05 prefill kernel)
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ out, const float* __restrict__ gate, int ldg, int M, int H, int Dv) {
  const size_t total = (size_t)M * H * Dv;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t mh = i / Dv;
    out[i] = from_f<T>(to_f(out[i]) * sigmoid_f(gate[(mh / H) * ldg + mh % H]));
  }
}

}  // namespace jl

using namespace jl;

extern "C" JL_API int jl_attn_prep(const float* y, int ldy, int q_off, int k_off, int v_off, void* q_out, void* k_cache,
                                   void* v_cache, const float* cos_t, const float* sin_t, int max_pos, int rot, int unit_norm,
                                   float eps, const int* cache_len, const int* pad_left, int B, int S, int H, int G, int D, int Dv,
                                   int T_cap, int dtype, void* stream) {
  JL_CHECK_ARG(B >= 1 && S >= 1 && H >= 1 && G >= 1 && D >= 1 && Dv >= 1, "jl_attn_prep: bad shape");
  JL_CHECK_ARG(rot >= 0 && rot <= D && rot % 2 == 0, "jl_attn_prep: rot=%d must be even and <= D=%d", rot, D);
  JL_CHECK_ARG(k_off >= 0 || (k_cache == nullptr && v_cache == nullptr), "jl_attn_prep: queries-only call takes no caches");
  PrepParams p{y, ldy, q_off, k_off, v_off, B, S, H, G, D, Dv, T_cap, rot, cos_t, sin_t, max_pos, unit_norm, eps, cache_len, pad_left};
  const int n_heads = k_off >= 0 ? H + 2 * G : H;
  const int pair_loads = D % 2 == 0 && ldy % 2 == 0 && q_off % 2 == 0 && (k_off < 0 || k_off % 2 == 0) && (uintptr_t)y % 8 == 0;
  dim3 grid(B * S, (n_heads + AP_WARPS - 1) / AP_WARPS);
  count_launch();
  JL_DISPATCH_DTYPE(dtype, attn_prep_kernel<T><<<grid, AP_WARPS * 32, 0, (cudaStream_t)stream>>>(p, (T*)q_out, (T*)k_cache,
                                                                                                (T*)v_cache, n_heads, pair_loads));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_attn_generic(const void* q, const void* k_cache, const void* v_cache, void* out, const float* gate, int ldg,
                                      const int* cache_len, const int* pad_left, int B, int S, int H, int G, int D, int Dv,
                                      int T_cap, float scale, int dtype, void* stream) {
  JL_CHECK_ARG(B >= 1 && S >= 1 && G >= 1 && H % G == 0, "jl_attn_generic: H=%d not a multiple of G=%d", H, G);
  JL_CHECK_ARG(Dv <= 32 * AT_MAXV, "jl_attn_generic: value size %d above %d", Dv, 32 * AT_MAXV);
  AttnParams p{B, S, H, G, D, Dv, T_cap, scale, cache_len, pad_left, gate, ldg};
  cudaStream_t st = (cudaStream_t)stream;
  count_launch();
  if (S == 1) {
    const size_t smem = (size_t)(D + 2 * AD_WARPS + AD_WARPS * Dv) * sizeof(float);
    JL_DISPATCH_DTYPE(dtype, attn_decode_kernel<T><<<dim3(H, B), AD_WARPS * 32, smem, st>>>(p, (const T*)q, (const T*)k_cache,
                                                                                         (const T*)v_cache, (T*)out));
  } else {
    const int nw = 4;
    const size_t smem = (size_t)nw * D * sizeof(float);
    JL_DISPATCH_DTYPE(dtype, attn_rows_kernel<T><<<dim3((S + nw - 1) / nw, H, B), nw * 32, smem, st>>>(
                                 p, (const T*)q, (const T*)k_cache, (const T*)v_cache, (T*)out));
  }
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}

extern "C" JL_API int jl_head_gate(void* out, const float* gate, int ldg, int M, int H, int Dv, int dtype, void* stream) {
  JL_CHECK_ARG(M >= 1 && H >= 1 && Dv >= 1, "jl_head_gate: bad shape");
  const size_t total = (size_t)M * H * Dv;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  count_launch();
  JL_DISPATCH_DTYPE(dtype, head_gate_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>((T*)out, gate, ldg, M, H, Dv));
  JL_CUDA(cudaGetLastError());
  return JL_OK;
}
