// Latent attention (mixers.h): every token caches one normed low-rank vector c [kv_rank] and one rotated key part
// kr [rot_dim] shared by all heads; a head's key is (W_uk c, kr) and its value W_uv c.  The kernels work in the latent
// space ("absorbed" form): the query is carried into it once per token, qlat_h = (W_uk,h^T q_h, rot(q_h,rot)), the scores
// are qlat_h . (c_j, kr_j), the softmax-weighted sum of the cached c_j is taken per head, and W_uv is applied to that
// sum afterwards — so neither prefill nor decode ever rebuilds per-head keys or values of the window, and both read the
// same paged cache rows [slot][kv_rank + rot_dim].  The two per-head projections are batched launches of linear.cu.
//
// Rotation: interleaved pairs (2i, 2i+1) of the first rot_dims of the rotated part, angles from a table computed in
// double.  Window: key j is visible from position p when 0 <= p - j < window.  Softmax statistics are fp32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <math.h>

#include <vector>

#include "mixers.h"

namespace b200 {
namespace {

typedef __nv_bfloat16 bf16;
__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float block_sum(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[wrp] = v;
  __syncthreads();
  float s = 0.f;
  for (int i = 0; i < nw; ++i) s += red[i];   // same order in every thread
  return s;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[wrp] = v;
  __syncthreads();
  float s = -FLT_MAX;
  for (int i = 0; i < nw; ++i) s = fmaxf(s, red[i]);
  return s;
}

// one CTA per token
template <typename T>
__global__ void __launch_bounds__(128) latent_prep_kernel(LatentPrepArgs a) {
  __shared__ float red[8];
  const int t = blockIdx.x;
  const int C = a.kv_rank, R = a.rot_dim, D = a.dim;
  const T* d = static_cast<const T*>(a.dkv) + static_cast<long long>(t) * a.lddkv;
  const int pos = a.positions[t];
  T* row = static_cast<T*>(a.cache) + static_cast<long long>(a.slots[t]) * (C + R);
  float ss = 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) { const float v = ldf(d + i); ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(C) + a.eps);
  for (int i = threadIdx.x; i < C; i += blockDim.x) stf(row + i, ldf(d + i) * inv * a.norm_w[i]);
  const int half = a.rot_dims / 2;
  const float2* cs = a.rope + static_cast<long long>(pos) * half;
  // shared rotated key part
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const int pr = i >> 1;
    float v = ldf(d + C + i);
    if (pr < half) {
      const float u0 = ldf(d + C + 2 * pr), u1 = ldf(d + C + 2 * pr + 1);
      const float2 c = cs[pr];
      v = (i & 1) ? fmaf(u1, c.x, u0 * c.y) : fmaf(u0, c.x, -u1 * c.y);
    }
    stf(row + C + i, v);
  }
  // rotated part of every query head -> tail of the latent query
  const T* q = static_cast<const T*>(a.q) + static_cast<long long>(t) * a.ldq;
  float* ql = a.qlat + static_cast<long long>(t) * a.heads * (C + R);
  for (int e = threadIdx.x; e < a.heads * R; e += blockDim.x) {
    const int h = e / R, i = e - h * R, pr = i >> 1;
    const T* qr = q + h * (D + R) + D;
    float v = ldf(qr + i);
    if (pr < half) {
      const float u0 = ldf(qr + 2 * pr), u1 = ldf(qr + 2 * pr + 1);
      const float2 c = cs[pr];
      v = (i & 1) ? fmaf(u1, c.x, u0 * c.y) : fmaf(u0, c.x, -u1 * c.y);
    }
    ql[h * (C + R) + C + i] = v;
  }
}

// one CTA per (token, head); dynamic shared memory: qlat row [C + R] + scores [window]
template <typename T>
__global__ void __launch_bounds__(128) latent_attn_kernel(LatentAttnArgs a) {
  extern __shared__ float sm[];
  __shared__ float red[8];
  const int t = blockIdx.x, h = blockIdx.y;
  const int C = a.kv_rank, E = a.kv_rank + a.rot_dim;
  float* qs = sm;
  float* sc = sm + E;
  const int p = a.positions[t];
  const int lo = max(0, p - a.window + 1);
  const int nk = p - lo + 1;
  const int* bt = a.block_tables + static_cast<long long>(a.seq_of_tok[t]) * a.max_blocks;
  const T* cache = static_cast<const T*>(a.cache);
  const float* ql = a.qlat + (static_cast<long long>(t) * a.heads + h) * E;
  for (int i = threadIdx.x; i < E; i += blockDim.x) qs[i] = ql[i];
  __syncthreads();
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float mx = -FLT_MAX;
  for (int jj = wrp; jj < nk; jj += nw) {
    const int j = lo + jj;
    const T* kr = cache + (static_cast<long long>(bt[j / a.page]) * a.page + j % a.page) * E;
    float s = 0.f;
    for (int i = lane; i < E; i += 32) s = fmaf(qs[i], ldf(kr + i), s);
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    s *= a.scale;
    if (lane == 0) sc[jj] = s;
    mx = fmaxf(mx, s);
  }
  mx = block_max(mx, red);   // includes the barrier that publishes sc[]
  float sum = 0.f;
  for (int jj = threadIdx.x; jj < nk; jj += blockDim.x) {
    const float e = expf(sc[jj] - mx);
    sc[jj] = e;
    sum += e;
  }
  sum = block_sum(sum, red);
  const float inv = 1.0f / sum;
  float* out = a.olat + (static_cast<long long>(t) * a.heads + h) * C;
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    float acc = 0.f;
    for (int jj = 0; jj < nk; ++jj) {
      const int j = lo + jj;
      const T* kr = cache + (static_cast<long long>(bt[j / a.page]) * a.page + j % a.page) * E;
      acc = fmaf(sc[jj], ldf(kr + i), acc);
    }
    out[i] = acc * inv;
  }
}

}  // namespace

int rope_table_interleaved(float2* table, int max_pos, int dims, double base, cudaStream_t st) {
  const int half = dims / 2;
  if (max_pos <= 0 || half <= 0) return 0;
  std::vector<float2> h(static_cast<size_t>(max_pos) * half);
  for (int i = 0; i < half; ++i) {
    const double f = pow(base, -2.0 * i / dims);
    for (int p = 0; p < max_pos; ++p) {
      const double ang = p * f;
      h[static_cast<size_t>(p) * half + i] = make_float2(static_cast<float>(cos(ang)), static_cast<float>(sin(ang)));
    }
  }
  if (cudaMemcpyAsync(table, h.data(), h.size() * sizeof(float2), cudaMemcpyHostToDevice, st) != cudaSuccess) return -2;
  return cudaStreamSynchronize(st) == cudaSuccess ? 0 : -2;
}

int latent_prep(const LatentPrepArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  if (a.rot_dims > a.rot_dim || a.rot_dims % 2) return -1;
  if (a.t == DT_BF16) latent_prep_kernel<bf16><<<a.T, 128, 0, st>>>(a);
  else latent_prep_kernel<float><<<a.T, 128, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int latent_attention(const LatentAttnArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  if (a.window < 1) return -1;
  const size_t smem = static_cast<size_t>(a.kv_rank + a.rot_dim + a.window) * sizeof(float);
  if (smem > 200 * 1024) return -1;
  dim3 grid(a.T, a.heads);
  if (a.t == DT_BF16) {
    if (smem > 48 * 1024 && cudaFuncSetAttribute(latent_attn_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) return -2;
    latent_attn_kernel<bf16><<<grid, 128, smem, st>>>(a);
  } else {
    if (smem > 48 * 1024 && cudaFuncSetAttribute(latent_attn_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) return -2;
    latent_attn_kernel<float><<<grid, 128, smem, st>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace b200
