// Softmax attention with grouped key/value heads over a paged cache, a sliding window and kept first tokens
// (mixers.h WindowAttnArgs), with the preparation in front of it: interleaved rotary positions under YaRN-style
// frequency scaling and a weightless unit-RMS norm of every query and key head (QkPrepArgs).
//
// Visibility of key j for the token at position p: j <= p and (p - j < window or j < keep_first).  The visible keys of
// a token are therefore two runs, [0, min(keep_first, lo)) and [lo, p] with lo = max(0, p - window + 1); both kernels
// walk exactly those and nothing else, in an order that depends only on p, so the result does not depend on how a
// prompt was cut into steps or on what shares the batch.  Kept tokens keep their own positions: keys are rotated once,
// when they are written, and never again.
//
// Kernels: `qk_prep_kernel` (one CTA per token: rotate, normalise, write the cache row), `window_attn_kernel` (any head
// size, bf16 or fp32 cache: one CTA per (token, head), four warps share the token's keys in 32-key chunks, a lane owns
// one key for the scores and a slice of the value columns for the output, online softmax in fp32, the warps' partial
// results meet in shared memory in a fixed order; the sigmoid output gate and the branch scale are applied before the
// single rounding to the storage type).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <math.h>
#include <stdlib.h>

#include <algorithm>
#include <vector>

#include "mixers.h"

namespace b200 {
namespace {

typedef __nv_bfloat16 bf16;
__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

// ---------------------------------------------------------------------------------------------- rotation, norm, cache write
// One CTA per token; a warp takes the heads u = warp, warp + nwarps, ...: u < heads is a query head, the next kv_heads are
// key heads.  A lane owns the dimension pairs (2i, 2i + 1), i = lane, lane + 32, ...; the odd last dimension of an odd dim is
// lane 0's.  Value rows are copied by all threads.
template <typename T>
__global__ void __launch_bounds__(128) qk_prep_kernel(QkPrepArgs a) {
  const long long t = blockIdx.x;
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int p = a.positions[t];
  const long long slot = a.slots[t];
  const int D = a.dim, half = a.rot_dims / 2, pairs = D / 2;
  const float2* cs = a.rope + static_cast<long long>(p) * half;
  const long long crow = static_cast<long long>(a.kv_heads) * (D + a.vdim);
  T* cache = static_cast<T*>(a.cache) + slot * crow;
  for (int u = wrp; u < a.heads + a.kv_heads; u += nw) {
    const bool isq = u < a.heads;
    const T* src = isq ? static_cast<const T*>(a.q) + t * a.ld + static_cast<long long>(u) * D
                       : static_cast<const T*>(a.k) + t * a.ld + static_cast<long long>(u - a.heads) * D;
    // rotate, accumulate the sum of squares; the rotated values are recomputed in the second pass (cheaper than a spill)
    float ss = 0.f;
    for (int i = lane; i < pairs; i += 32) {
      float x0 = ldf(src + 2 * i), x1 = ldf(src + 2 * i + 1);
      if (i < half) {
        const float2 c = cs[i];
        const float r0 = x0 * c.x - x1 * c.y, r1 = x1 * c.x + x0 * c.y;
        x0 = r0; x1 = r1;
      }
      ss = fmaf(x0, x0, ss);
      ss = fmaf(x1, x1, ss);
    }
    if ((D & 1) && lane == 0) { const float x = ldf(src + D - 1); ss = fmaf(x, x, ss); }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = a.unit_norm ? 1.0f / sqrtf(ss / static_cast<float>(D) + a.eps) : 1.0f;
    for (int i = lane; i < pairs; i += 32) {
      float x0 = ldf(src + 2 * i), x1 = ldf(src + 2 * i + 1);
      if (i < half) {
        const float2 c = cs[i];
        const float r0 = x0 * c.x - x1 * c.y, r1 = x1 * c.x + x0 * c.y;
        x0 = r0; x1 = r1;
      }
      if (isq) {
        float* dst = a.qn + (t * a.heads + u) * D;
        dst[2 * i] = x0 * inv; dst[2 * i + 1] = x1 * inv;
      } else {
        T* dst = cache + static_cast<long long>(u - a.heads) * D;
        stf(dst + 2 * i, x0 * inv); stf(dst + 2 * i + 1, x1 * inv);
      }
    }
    if ((D & 1) && lane == 0) {
      const float x = ldf(src + D - 1) * inv;
      if (isq) a.qn[(t * a.heads + u) * D + D - 1] = x;
      else stf(cache + static_cast<long long>(u - a.heads) * D + D - 1, x);
    }
  }
  const T* v = static_cast<const T*>(a.v) + t * a.ld;
  T* vdst = cache + static_cast<long long>(a.kv_heads) * D;
  for (int i = threadIdx.x; i < a.kv_heads * a.vdim; i += blockDim.x) vdst[i] = v[i];
}

// ---------------------------------------------------------------------------------------------- attention, any head size
constexpr int kWarps = 4;
constexpr int kMaxVR = 8;   // value columns per lane: vdim <= 256

template <typename T>
__device__ __forceinline__ float dot_row(const float* q, const T* k, int D, bool vec) {
  float acc = 0.f;
  if (vec) {
    if constexpr (sizeof(T) == 2) {
      for (int d = 0; d < D; d += 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(k + d);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc = fmaf(q[d + 2 * i], __uint_as_float(u[i] << 16), acc);
          acc = fmaf(q[d + 2 * i + 1], __uint_as_float(u[i] & 0xffff0000u), acc);
        }
      }
    } else {
      for (int d = 0; d < D; d += 4) {
        const float4 v = *reinterpret_cast<const float4*>(k + d);
        acc = fmaf(q[d], v.x, acc); acc = fmaf(q[d + 1], v.y, acc); acc = fmaf(q[d + 2], v.z, acc); acc = fmaf(q[d + 3], v.w, acc);
      }
    }
  } else {
    for (int d = 0; d < D; ++d) acc = fmaf(q[d], ldf(k + d), acc);
  }
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) window_attn_kernel(WindowAttnArgs a, bool vec) {
  extern __shared__ float sm[];   // q [dim] | per warp: m, l, acc [vdim]
  const long long t = blockIdx.x / a.heads;
  const int h = blockIdx.x % a.heads;
  const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;
  const int D = a.dim, Dv = a.vdim;
  const int g = h / (a.heads / a.kv_heads);
  const int p = a.positions[t];
  const int* bt = a.block_tables + static_cast<long long>(a.seq_of_tok[t]) * a.max_blocks;
  const int lo = max(0, p - a.window + 1);
  const int nk = min(a.keep_first, lo);      // kept first tokens outside the window
  const int n = nk + (p - lo + 1);
  float* qs = sm;
  float* part = sm + ((D + 3) & ~3);
  for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = a.qn[(t * a.heads + h) * D + d] * a.scale;
  __syncthreads();
  const long long crow = static_cast<long long>(a.kv_heads) * (D + Dv);
  const T* cache = static_cast<const T*>(a.cache);
  const long long koff = static_cast<long long>(g) * D, voff = static_cast<long long>(a.kv_heads) * D + static_cast<long long>(g) * Dv;
  float m = -FLT_MAX, l = 0.f, acc[kMaxVR];
#pragma unroll
  for (int r = 0; r < kMaxVR; ++r) acc[r] = 0.f;
  for (int c0 = wrp * 32; c0 < n; c0 += kWarps * 32) {
    const int i = c0 + lane;
    long long row = -1;
    float s = -FLT_MAX;
    if (i < n) {
      const int j = i < nk ? i : lo + (i - nk);
      row = static_cast<long long>(bt[j / a.page]) * a.page + j % a.page;
      s = dot_row(qs, cache + row * crow + koff, D, vec);
    }
    float cm = s;
    for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
    const float mn = fmaxf(m, cm);
    const float corr = expf(m - mn);
    const float pr = i < n ? expf(s - mn) : 0.f;
    float ps = pr;
    for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
    l = fmaf(l, corr, ps);
    m = mn;
#pragma unroll
    for (int r = 0; r < kMaxVR; ++r) acc[r] *= corr;
    const int cn = min(32, n - c0);
    for (int kk = 0; kk < cn; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, pr, kk);
      const long long rk = __shfl_sync(0xffffffffu, row, kk);
      const T* vp = cache + rk * crow + voff;
#pragma unroll
      for (int r = 0; r < kMaxVR; ++r) {
        const int c = lane + 32 * r;
        if (c < Dv) acc[r] = fmaf(pk, ldf(vp + c), acc[r]);
      }
    }
  }
  // the warps' partial (m, l, acc) meet in shared memory and are merged in warp order
  float* mine = part + wrp * (Dv + 2);
  if (lane == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
  for (int r = 0; r < kMaxVR; ++r) {
    const int c = lane + 32 * r;
    if (c < Dv) mine[2 + c] = acc[r];
  }
  __syncthreads();
  float mm = -FLT_MAX;
  for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, part[w * (Dv + 2)]);
  float ll = 0.f;
  float f[kWarps];
  for (int w = 0; w < kWarps; ++w) {
    const float pm = part[w * (Dv + 2)];
    f[w] = pm == -FLT_MAX ? 0.f : expf(pm - mm);
    ll = fmaf(part[w * (Dv + 2) + 1], f[w], ll);
  }
  const float inv = 1.0f / ll;
  const T* gate = static_cast<const T*>(a.gate);
  T* y = static_cast<T*>(a.y) + t * a.ldy + static_cast<long long>(h) * Dv;
  for (int c = threadIdx.x; c < Dv; c += blockDim.x) {
    float o = 0.f;
    for (int w = 0; w < kWarps; ++w) o = fmaf(part[w * (Dv + 2) + 2 + c], f[w], o);
    o *= inv;
    if (gate) o *= sigmoidf_(ldf(gate + t * a.ldg + static_cast<long long>(h) * Dv + c));
    stf(y + c, o * a.out_scale);
  }
}

}  // namespace

int rope_table_yarn(float2* table, int max_pos, int dims, double base, const RopeYarn* yarn, cudaStream_t st) {
  const int half = dims / 2;
  if (max_pos <= 0 || half <= 0) return 0;
  if (!(base > 0.0) || (yarn && !(yarn->factor > 0.0 && yarn->original > 0.0 && yarn->fast > 0.0 && yarn->slow > 0.0))) return -1;
  const double pi = 3.14159265358979323846;
  double lo = 0, hi = 0, mag = 1.0;
  if (yarn) {
    auto at = [&](double turns) { return dims * log(yarn->original / (2.0 * pi * turns)) / (2.0 * log(base)); };
    lo = std::max(floor(at(yarn->fast)), 0.0);
    hi = std::min(ceil(at(yarn->slow)), static_cast<double>(dims - 1));
    mag = 0.1 * log(yarn->factor) + 1.0;
  }
  std::vector<float2> h(static_cast<size_t>(max_pos) * half);
  for (int i = 0; i < half; ++i) {
    double f = pow(base, -2.0 * i / dims);
    if (yarn) {
      const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
      f = f / yarn->factor * ramp + f * (1.0 - ramp);
    }
    for (int p = 0; p < max_pos; ++p) {
      const double ang = p * f;
      h[static_cast<size_t>(p) * half + i] = make_float2(static_cast<float>(cos(ang) * mag), static_cast<float>(sin(ang) * mag));
    }
  }
  if (cudaMemcpyAsync(table, h.data(), h.size() * sizeof(float2), cudaMemcpyHostToDevice, st) != cudaSuccess) return -2;
  return cudaStreamSynchronize(st) == cudaSuccess ? 0 : -2;
}

int qk_rope_norm_cache(const QkPrepArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  if (a.heads < 1 || a.kv_heads < 1 || a.dim < 1 || a.vdim < 1 || a.rot_dims < 0 || a.rot_dims > a.dim || a.rot_dims % 2 || (a.rot_dims && !a.rope)) return -1;
  if (a.t == DT_BF16) qk_prep_kernel<bf16><<<a.T, 128, 0, st>>>(a);
  else qk_prep_kernel<float><<<a.T, 128, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int window_attention(const WindowAttnArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  if (a.heads < 1 || a.kv_heads < 1 || a.heads % a.kv_heads || a.dim < 1 || a.vdim < 1 || a.vdim > 32 * kMaxVR || a.window < 1 || a.keep_first < 0 ||
      a.page < 1) return -1;
  const size_t es = dtype_bytes(a.t);
  const int vl = a.t == DT_BF16 ? 8 : 4;
  const bool vec = a.dim % vl == 0 && (static_cast<long long>(a.kv_heads) * (a.dim + a.vdim)) % vl == 0 && reinterpret_cast<uintptr_t>(a.cache) % 16 == 0;
  (void)es;
  const size_t smem = (static_cast<size_t>((a.dim + 3) & ~3) + kWarps * (a.vdim + 2)) * sizeof(float);
  if (smem > 48 * 1024) return -1;
  const unsigned grid = static_cast<unsigned>(static_cast<long long>(a.T) * a.heads);
  if (a.t == DT_BF16) window_attn_kernel<bf16><<<grid, kWarps * 32, smem, st>>>(a, vec);
  else window_attn_kernel<float><<<grid, kWarps * 32, smem, st>>>(a, vec);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace b200
