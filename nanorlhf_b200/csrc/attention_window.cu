// Sliding-window attention over the paged KV cache, for prompt portions and decoded tokens alike: the keys of a step's own
// tokens are written to their pages first (nrl_qknorm_kv_write), then every token reads the last `window` keys of its
// sequence through the block table, so the result does not depend on how the sequence was cut into steps.
// Query / key sizes (D) and value size (Dv) are independent runtime values; scores, softmax and the output sum are float.
// Compiled WITHOUT fast-math.
#include <cuda_bf16.h>

#include "hybrid_kernels.h"

namespace {

__device__ __forceinline__ float ld(const float* p, long i) { return p[i]; }
__device__ __forceinline__ float ld(const __nv_bfloat16* p, long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st(float* p, long i, float v) { p[i] = v; }
__device__ __forceinline__ void st(__nv_bfloat16* p, long i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// warp per (token, head): heads 0..Hq-1 are queries (normalised in place), Hq..Hq+Hkv-1 keys (normalised into the cache),
// then Hkv value heads (copied into the cache)
template <typename CT>
__global__ void qknorm_kv_write_kernel(float* __restrict__ q, long sq, const float* __restrict__ k, long sk, const float* __restrict__ v,
                                       long sv, const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                                       CT* __restrict__ k_cache, CT* __restrict__ v_cache, const int* __restrict__ kv_slot, long T,
                                       int Hq, int Hkv, int D, int Dv, int page) {
  const long wid = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int per = Hq + 2 * Hkv;
  if (wid >= T * per) return;
  const long t = wid / per;
  const int hh = static_cast<int>(wid - t * per);
  const int slot = kv_slot[t];
  const long pg = slot / page, off = slot % page;
  if (hh < Hq) {
    float* x = q + t * sq + static_cast<long>(hh) * D;
    float ss = 0.f;
    for (int c = lane; c < D; c += 32) ss += x[c] * x[c];
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / static_cast<float>(D) + eps);
    for (int c = lane; c < D; c += 32) x[c] = x[c] * r * qw[c];
  } else if (hh < Hq + Hkv) {
    const int g = hh - Hq;
    const float* x = k + t * sk + static_cast<long>(g) * D;
    float ss = 0.f;
    for (int c = lane; c < D; c += 32) ss += x[c] * x[c];
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / static_cast<float>(D) + eps);
    CT* dst = k_cache + ((pg * Hkv + g) * page + off) * D;
    for (int c = lane; c < D; c += 32) st(dst, c, x[c] * r * kw[c]);
  } else {
    const int g = hh - Hq - Hkv;
    const float* x = v + t * sv + static_cast<long>(g) * Dv;
    CT* dst = v_cache + ((pg * Hkv + g) * page + off) * Dv;
    for (int c = lane; c < Dv; c += 32) st(dst, c, x[c]);
  }
}

constexpr int kWarps = 4;
constexpr int kMaxDvPerLane = 8;       // Dv <= 256

// block per (token, query head); the window's keys are dealt to the warps in runs of 32 (one key per lane)
template <typename CT, typename OT>
__global__ void window_attention_kernel(const float* __restrict__ q, long sq, const CT* __restrict__ k_cache,
                                        const CT* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
                                        const int* __restrict__ tok_entry, const int* __restrict__ pos, int window, float scale,
                                        float out_scale, OT* __restrict__ out, long so, int Hq, int Hkv, int D, int Dv, int page) {
  extern __shared__ float sm[];
  float* sq_ = sm;                               // [D]
  float* accs = sq_ + D;                         // [kWarps][Dv]
  float* ml = accs + kWarps * Dv;                // [kWarps][2]
  const long t = blockIdx.x;
  const int h = blockIdx.y, g = h / (Hq / Hkv);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int p = pos[t];
  const int* bt = block_table + static_cast<long>(tok_entry[t]) * max_blocks;
  for (int c = threadIdx.x; c < D; c += blockDim.x) sq_[c] = q[t * sq + static_cast<long>(h) * D + c];
  __syncthreads();
  const int lo = p - window + 1 > 0 ? p - window + 1 : 0;
  const int nkeys = p - lo + 1;
  float m = -INFINITY, l = 0.f;
  float acc[kMaxDvPerLane];
#pragma unroll
  for (int i = 0; i < kMaxDvPerLane; ++i) acc[i] = 0.f;
  for (int base = w * 32; base < nkeys; base += kWarps * 32) {
    const int j = lo + base + lane;
    const bool ok = base + lane < nkeys;
    float sc = -INFINITY;
    long vrow = 0;
    if (ok) {
      const long pg = bt[j / page];
      const long cell = (pg * Hkv + g) * page + (j % page);
      const CT* kr = k_cache + cell * D;
      float d = 0.f;
      for (int c = 0; c < D; ++c) d += sq_[c] * ld(kr, c);
      sc = d * scale;
      vrow = cell * Dv;
    }
    const float mn = fmaxf(m, warp_max(sc));
    const float corr = expf(m - mn);               // m = -inf on the first run: exp(-inf) = 0
    const float pr = ok ? expf(sc - mn) : 0.f;
    l = l * corr + warp_sum(pr);
#pragma unroll
    for (int i = 0; i < kMaxDvPerLane; ++i) acc[i] *= corr;
    const int cnt = nkeys - base < 32 ? nkeys - base : 32;
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, pr, jj);
      const long vr = __shfl_sync(0xffffffffu, vrow, jj);
#pragma unroll
      for (int i = 0; i < kMaxDvPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c < Dv) acc[i] += pj * ld(v_cache, vr + c);
      }
    }
    m = mn;
  }
#pragma unroll
  for (int i = 0; i < kMaxDvPerLane; ++i) {
    const int c = lane + 32 * i;
    if (c < Dv) accs[w * Dv + c] = acc[i];
  }
  if (lane == 0) {
    ml[2 * w] = m;
    ml[2 * w + 1] = l;
  }
  __syncthreads();
  float mt = -INFINITY;
  for (int i = 0; i < kWarps; ++i) mt = fmaxf(mt, ml[2 * i]);
  float lt = 0.f, f[kWarps];
  for (int i = 0; i < kWarps; ++i) {
    f[i] = ml[2 * i] == -INFINITY ? 0.f : expf(ml[2 * i] - mt);
    lt += f[i] * ml[2 * i + 1];
  }
  for (int c = threadIdx.x; c < Dv; c += blockDim.x) {
    float a = 0.f;
    for (int i = 0; i < kWarps; ++i) a += f[i] * accs[i * Dv + c];
    st(out, t * so + static_cast<long>(h) * Dv + c, out_scale * (a / lt));
  }
}

}  // namespace

extern "C" {

cudaError_t nrl_qknorm_kv_write(float* q, long sq, const float* k, long sk, const float* v, long sv, const float* qw, const float* kw,
                                float eps, void* k_cache, void* v_cache, int cache_f32, const int* kv_slot, int T, int Hq, int Hkv,
                                int D, int Dv, int page, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  const long warps = static_cast<long>(T) * (Hq + 2 * Hkv);
  const unsigned blocks = static_cast<unsigned>((warps + 3) / 4);
  if (cache_f32)
    qknorm_kv_write_kernel<float><<<blocks, 128, 0, s>>>(q, sq, k, sk, v, sv, qw, kw, eps, static_cast<float*>(k_cache),
                                                         static_cast<float*>(v_cache), kv_slot, T, Hq, Hkv, D, Dv, page);
  else
    qknorm_kv_write_kernel<__nv_bfloat16><<<blocks, 128, 0, s>>>(q, sq, k, sk, v, sv, qw, kw, eps,
                                                                 static_cast<__nv_bfloat16*>(k_cache),
                                                                 static_cast<__nv_bfloat16*>(v_cache), kv_slot, T, Hq, Hkv, D, Dv, page);
  return cudaGetLastError();
}

cudaError_t nrl_window_attention(const float* q, long sq, const void* k_cache, const void* v_cache, int cache_f32,
                                 const int* block_table, int max_blocks, const int* tok_entry, const int* pos, int window,
                                 float scale, float out_scale, void* out, long so, int out_f32, int T, int Hq, int Hkv, int D, int Dv,
                                 int page, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (Dv > 32 * kMaxDvPerLane || Hq % Hkv != 0 || window < 1 || cache_f32 != out_f32) return cudaErrorInvalidValue;
  const size_t smem = sizeof(float) * (D + kWarps * Dv + 2 * kWarps);
  if (smem > 48 * 1024) return cudaErrorInvalidValue;
  const dim3 grid(T, Hq);
  if (cache_f32)
    window_attention_kernel<float, float><<<grid, kWarps * 32, smem, s>>>(
        q, sq, static_cast<const float*>(k_cache), static_cast<const float*>(v_cache), block_table, max_blocks, tok_entry, pos, window,
        scale, out_scale, static_cast<float*>(out), so, Hq, Hkv, D, Dv, page);
  else
    window_attention_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, kWarps * 32, smem, s>>>(
        q, sq, static_cast<const __nv_bfloat16*>(k_cache), static_cast<const __nv_bfloat16*>(v_cache), block_table, max_blocks,
        tok_entry, pos, window, scale, out_scale, static_cast<__nv_bfloat16*>(out), so, Hq, Hkv, D, Dv, page);
  return cudaGetLastError();
}

}  // extern "C"
