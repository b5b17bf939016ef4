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

#include <stdlib.h>

#include <algorithm>
#include <atomic>
#include <vector>

#include "launch.h"
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

// ---------------------------------------------------------------- tensor-core kernel (bf16 cache)
// One CTA = 16 query rows = TQ consecutive tokens of one sequence x HB heads (HB = min(heads, 16), TQ = 16 / HB), 8 warps.
// The window of the tile's tokens is walked in tiles of 64 keys, gathered from the pages into shared memory by cp.async
// (double buffered).  Per key tile: warp w multiplies the 16 latent queries with its 8 keys over the whole latent width
// (mma.sync m16n8k16, fragments by ldmatrix), the scores go through shared memory to a 256-thread online-softmax pass
// (fp32 running maximum and sum per row, window and causal mask per row), and every warp then accumulates its own
// columns of sum_j p_j c_j from the same key tile (ldmatrix.trans), rescaled when a row's maximum moves.
constexpr int kKeys = 64;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ldsm_x4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kMaxPairs = 4;   // 16-column pairs of the latent value width per warp: kv_rank <= 8 * 4 * 16 = 512

// MB = 16-row blocks per CTA: two for steps made of prompt portions (each key tile then serves twice the rows)
template <int MB>
__global__ void __launch_bounds__(256) latent_attn_mma_kernel(LatentAttnArgs a, const int* seqs, int nseq, int TQ, int HB, int nsplit, float* split_ws) {
  extern __shared__ __align__(16) unsigned char smraw[];
  constexpr int R = 16 * MB;
  const int C = a.kv_rank, E = a.kv_rank + a.rot_dim, LDE = E + 8;
  bf16* Qs = reinterpret_cast<bf16*>(smraw);                       // [R][LDE]
  bf16* Ks = Qs + R * LDE;                                         // [2][kKeys][LDE]
  float* Ss = reinterpret_cast<float*>(Ks + 2 * kKeys * LDE);      // [R][kKeys + 4]
  bf16* Ps = reinterpret_cast<bf16*>(Ss + R * (kKeys + 4));        // [R][kKeys + 8]
  float* Ms = reinterpret_cast<float*>(Ps + R * (kKeys + 8));      // running max [R], sum [R], rescale [R]
  float* Ls = Ms + R;
  float* As = Ls + R;
  // which (sequence, token tile) is this CTA's
  int idx = blockIdx.x, seq = -1, tile = 0;
  for (int s = 0; s < nseq; ++s) {
    const int tiles = (seqs[s * 8 + 1] + TQ - 1) / TQ;
    if (idx < tiles) { seq = s; tile = idx; break; }
    idx -= tiles;
  }
  if (seq < 0) return;
  const int tok0 = seqs[seq * 8 + 0], n = seqs[seq * 8 + 1], pos0 = seqs[seq * 8 + 2];
  const int tq0 = tile * TQ, ntq = min(TQ, n - tq0);
  const int h0 = blockIdx.y * HB;
  const int p_first = pos0 + tq0, p_last = p_first + ntq - 1;
  const int lo = max(0, p_first - a.window + 1);
  const int all_tiles = (p_last - lo) / kKeys + 1;
  // split form (few sequences, long windows): CTA z of nsplit walks its share of the key tiles and leaves an unnormalised partial
  const int per = (all_tiles + nsplit - 1) / nsplit;
  const int t_begin = min(all_tiles, static_cast<int>(blockIdx.z) * per), t_end = min(all_tiles, t_begin + per);
  const int* bt = a.block_tables + static_cast<long long>(seq) * a.max_blocks;
  const bf16* cache = static_cast<const bf16*>(a.cache);
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int chunks = E / 8;   // 16-byte pieces of one cache row

  // four threads per key row: one block-table lookup per thread and tile, then its 16-byte pieces at a fixed stride
  auto load_tile = [&](int ti, int buf) {
    const int jt = tid >> 2, sub = tid & 3;
    const int j = lo + ti * kKeys + jt;
    bf16* d = Ks + (static_cast<size_t>(buf) * kKeys + jt) * LDE;
    if (j <= p_last) {
      const bf16* src = cache + (static_cast<long long>(bt[j / a.page]) * a.page + j % a.page) * E;
      for (int c = sub; c < chunks; c += 4) cp_async16(smem_addr(d + c * 8), src + c * 8);
    } else {
      for (int c = sub; c < chunks; c += 4) *reinterpret_cast<uint4*>(d + c * 8) = make_uint4(0, 0, 0, 0);
    }
  };
  if (t_begin < t_end) load_tile(t_begin, t_begin & 1);
  // latent queries of the R rows (row r = token tq0 + r / HB, head h0 + r % HB), rounded to bf16
  {
    const int e4 = E / 4;   // float4 pieces per row (E is a multiple of 16)
#pragma unroll 4
    for (int e = tid; e < R * e4; e += 256) {
      const int r = e / e4, c = (e - r * e4) * 4, tq = r / HB, h = h0 + r % HB;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tq < ntq && h < a.heads) v = __ldg(reinterpret_cast<const float4*>(a.qlat + (static_cast<long long>(tok0 + tq0 + tq) * a.heads + h) * E + c));
      *reinterpret_cast<__nv_bfloat162*>(Qs + r * LDE + c) = __floats2bfloat162_rn(v.x, v.y);
      *reinterpret_cast<__nv_bfloat162*>(Qs + r * LDE + c + 2) = __floats2bfloat162_rn(v.z, v.w);
    }
  }
  if (tid < R) { Ms[tid] = -FLT_MAX; Ls[tid] = 0.f; As[tid] = 1.f; }
  float acc[MB][kMaxPairs][2][4];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int i = 0; i < kMaxPairs; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[mb][i][j][k] = 0.f;
  const int npairs = C / 16;
  const int g = lane >> 2, t4 = lane & 3;

  for (int ti = t_begin; ti < t_end; ++ti) {
    cp_async_wait_all();
    __syncthreads();
    if (ti + 1 < t_end) load_tile(ti + 1, (ti + 1) & 1);
    const bf16* Kt = Ks + static_cast<size_t>(ti & 1) * kKeys * LDE;
    // ---- scores of this warp's 8 keys, for every row block
    {
      // two accumulators per row block (even / odd k-steps): the dependent mma chain is half as long
      float c[MB][4], c2[MB][4];
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int i = 0; i < 4; ++i) c[mb][i] = c2[mb][i] = 0.f;
      const uint32_t qa = smem_addr(Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LDE + 8 * (lane >> 4));
      const uint32_t ka = smem_addr(Kt + (8 * w + (lane & 7)) * LDE + 8 * (lane >> 3));
      for (int ks = 0; ks < E; ks += 32) {
        uint32_t bq[4];
        ldsm_x4(bq, ka + ks * 2);   // keys x k [ks, ks + 32): b0, b1 of two k-steps
        const bool two = ks + 16 < E;
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          uint32_t a0[4];
          ldsm_x4(a0, qa + (mb * 16 * LDE + ks) * 2);
          mma16816(c[mb], a0, bq[0], bq[1]);
          if (two) {
            uint32_t a1[4];
            ldsm_x4(a1, qa + (mb * 16 * LDE + ks + 16) * 2);
            mma16816(c2[mb], a1, bq[2], bq[3]);
          }
        }
      }
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int i = 0; i < 4; ++i) c[mb][i] += c2[mb][i];
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        float* sp = Ss + (mb * 16 + g) * (kKeys + 4) + 8 * w + 2 * t4;
        sp[0] = c[mb][0]; sp[1] = c[mb][1];
        sp[8 * (kKeys + 4)] = c[mb][2]; sp[8 * (kKeys + 4) + 1] = c[mb][3];
      }
    }
    __syncthreads();
    // ---- online softmax: thread -> (row, 4 keys)
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
      const int srow = mb * 16 + (tid >> 4), sk = (tid & 15) * 4;
      const int s_tq = srow / HB;
      const bool s_valid = s_tq < ntq && h0 + srow % HB < a.heads;
      const int s_pos = p_first + s_tq;
      const int j0 = lo + ti * kKeys + sk;
      float sv[4], mx = -FLT_MAX;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = j0 + i;
        const bool vis = s_valid && j <= s_pos && j > s_pos - a.window;
        sv[i] = vis ? Ss[srow * (kKeys + 4) + sk + i] * a.scale : -FLT_MAX;
        mx = fmaxf(mx, sv[i]);
      }
      const float m_old = Ms[srow];
      for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      float pv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { pv[i] = sv[i] == -FLT_MAX ? 0.f : expf(sv[i] - m_new); sum += pv[i]; }
      for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      *reinterpret_cast<__nv_bfloat162*>(Ps + srow * (kKeys + 8) + sk) = __floats2bfloat162_rn(pv[0], pv[1]);
      *reinterpret_cast<__nv_bfloat162*>(Ps + srow * (kKeys + 8) + sk + 2) = __floats2bfloat162_rn(pv[2], pv[3]);
      if ((tid & 15) == 0) {
        const float al = m_old == -FLT_MAX ? 0.f : expf(m_old - m_new);
        Ms[srow] = m_new;
        Ls[srow] = Ls[srow] * al + sum;
        As[srow] = m_new == -FLT_MAX ? 1.f : al;
      }
    }
    __syncthreads();
    // ---- values: this warp's column pairs, for every row block
    {
      uint32_t pa[MB][4][4];
      float al0[MB], al1[MB];
      const uint32_t pbase = smem_addr(Ps + ((lane & 7) + 8 * ((lane >> 3) & 1)) * (kKeys + 8) + 8 * (lane >> 4));
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        al0[mb] = As[mb * 16 + g];
        al1[mb] = As[mb * 16 + g + 8];
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) ldsm_x4(pa[mb][ks], pbase + (mb * 16 * (kKeys + 8) + ks * 16) * 2);
      }
#pragma unroll
      for (int i = 0; i < kMaxPairs; ++i) {
        const int pp = w + 8 * i;
        if (pp < npairs) {
#pragma unroll
          for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int j = 0; j < 2; ++j) { acc[mb][i][j][0] *= al0[mb]; acc[mb][i][j][1] *= al0[mb]; acc[mb][i][j][2] *= al1[mb]; acc[mb][i][j][3] *= al1[mb]; }
          const uint32_t vb = smem_addr(Kt + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LDE + 16 * pp + 8 * (lane >> 4));
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            uint32_t bv[4];
            ldsm_x4_trans(bv, vb + ks * 16 * LDE * 2);
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
              mma16816(acc[mb][i][0], pa[mb][ks], bv[0], bv[1]);
              mma16816(acc[mb][i][1], pa[mb][ks], bv[2], bv[3]);
            }
          }
        }
      }
    }
  }
  __syncthreads();
  // ---- normalise and store: rows g and g + 8 of every row block
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = mb * 16 + g + 8 * half, tq = r / HB, h = h0 + r % HB;
      if (tq >= ntq || h >= a.heads) continue;
      const long long orow = static_cast<long long>(tok0 + tq0 + tq) * a.heads + h;
      float inv = 1.0f / Ls[r];
      float* out = a.olat + orow * C;
      if (nsplit > 1) {
        // partial: [row][split][C + 2] = unnormalised sums, running maximum, running sum
        out = split_ws + (orow * nsplit + blockIdx.z) * (C + 2);
        inv = 1.0f;
        if (w == 0 && t4 == 0) { out[C] = Ms[r]; out[C + 1] = Ls[r]; }
      }
#pragma unroll
      for (int i = 0; i < kMaxPairs; ++i) {
        const int pp = w + 8 * i;
        if (pp < npairs) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            *reinterpret_cast<float2*>(out + 16 * pp + 8 * j + 2 * t4) = make_float2(acc[mb][i][j][2 * half] * inv, acc[mb][i][j][2 * half + 1] * inv);
          }
        }
      }
    }
}

// one warp per (token, head): combine the splits' partials
__global__ void latent_attn_merge_kernel(const float* ws, float* olat, int C, int nsplit, long long rows) {
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float* p = ws + row * nsplit * (C + 2);
  float M = -FLT_MAX;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, p[s * (C + 2) + C]);
  float L = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float m = p[s * (C + 2) + C];
    if (m != -FLT_MAX) L += p[s * (C + 2) + C + 1] * expf(m - M);
  }
  const float inv = 1.0f / L;
  for (int c = lane; c < C; c += 32) {
    float acc = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float m = p[s * (C + 2) + C];
      if (m != -FLT_MAX) acc = fmaf(p[s * (C + 2) + c], expf(m - M), acc);
    }
    olat[row * C + c] = acc * inv;
  }
}

// ---------------------------------------------------------------- wide form for long prompt portions
// 64 query rows per CTA (TQ = 64 / HB tokens x HB heads) against key tiles of 32: every key row fetched from the pages
// serves twice the rows of the 32-row form, and every value fragment read from shared memory feeds eight mma instead of
// four.  Scores: warp w owns row block w % 4 and key half w / 4 (16 x 16 per k-step: one query and one key ldmatrix for two
// mma).  Softmax: four threads per row, eight keys each.  Values: warp w owns the same column pairs as above, for all four
// row blocks.  No split form: steps that take this kernel have CTAs enough.
constexpr int kWideKeys = 32;
constexpr int kWideRows = 64;

__global__ void __launch_bounds__(256) latent_attn_mma_wide_kernel(LatentAttnArgs a, const int* seqs, int nseq, int TQ, int HB, int NST) {
  extern __shared__ __align__(16) unsigned char smraw[];
  constexpr int R = kWideRows, MB = R / 16, KT = kWideKeys, LDS = KT + 4, LDP = KT + 8;
  const int C = a.kv_rank, E = a.kv_rank + a.rot_dim, LDE = E + 8;
  bf16* Qs = reinterpret_cast<bf16*>(smraw);                  // [R][LDE]
  bf16* Ks = Qs + R * LDE;                                    // [NST][KT][LDE], NST = 2 or 3 key tiles in flight
  float* Ss = reinterpret_cast<float*>(Ks + NST * KT * LDE);  // [R][LDS]
  bf16* Ps = reinterpret_cast<bf16*>(Ss + R * LDS);           // [R][LDP]
  float* Ms = reinterpret_cast<float*>(Ps + R * LDP);         // running max [R], sum [R], rescale [R]
  float* Ls = Ms + R;
  float* As = Ls + R;
  int idx = blockIdx.x, seq = -1, tile = 0;
  for (int s = 0; s < nseq; ++s) {
    const int tiles = (seqs[s * 8 + 1] + TQ - 1) / TQ;
    if (idx < tiles) { seq = s; tile = idx; break; }
    idx -= tiles;
  }
  if (seq < 0) return;
  const int tok0 = seqs[seq * 8 + 0], n = seqs[seq * 8 + 1], pos0 = seqs[seq * 8 + 2];
  const int tq0 = tile * TQ, ntq = min(TQ, n - tq0);
  const int h0 = blockIdx.y * HB;
  const int p_first = pos0 + tq0, p_last = p_first + ntq - 1;
  const int lo = max(0, p_first - a.window + 1);
  const int ntiles = (p_last - lo) / KT + 1;
  const int* bt = a.block_tables + static_cast<long long>(seq) * a.max_blocks;
  const bf16* cache = static_cast<const bf16*>(a.cache);
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int chunks = E / 8;   // 16-byte pieces of one cache row

  // eight threads per key row: one block-table lookup per thread and tile, read one tile ahead of its use (tiles are
  // loaded in order), so that the copies of a tile are not issued behind a dependent global load
  int blk_next = 0;
  {
    const int j = lo + (tid >> 3);
    if (j <= p_last) blk_next = bt[j / a.page];
  }
  auto load_tile = [&](int ti, int buf) {
    const int jt = tid >> 3, sub = tid & 7;
    const int j = lo + ti * KT + jt;
    bf16* d = Ks + (static_cast<size_t>(buf) * KT + jt) * LDE;
    const int blk = blk_next;
    if (j + KT <= p_last) blk_next = bt[(j + KT) / a.page];
    if (j <= p_last) {
      const bf16* src = cache + (static_cast<long long>(blk) * a.page + j % a.page) * E;
      for (int c = sub; c < chunks; c += 8) cp_async16(smem_addr(d + c * 8), src + c * 8);
    } else {
      for (int c = sub; c < chunks; c += 8) *reinterpret_cast<uint4*>(d + c * 8) = make_uint4(0, 0, 0, 0);
    }
  };
  for (int t = 0; t < NST - 1; ++t) {
    if (t < ntiles) load_tile(t, t);
    cp_async_commit();
  }
  {
    const int e4 = E / 4;
#pragma unroll 12
    for (int e = tid; e < R * e4; e += 256) {
      const int r = e / e4, c = (e - r * e4) * 4, tq = r / HB, h = h0 + r % HB;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tq < ntq && h < a.heads) v = __ldg(reinterpret_cast<const float4*>(a.qlat + (static_cast<long long>(tok0 + tq0 + tq) * a.heads + h) * E + c));
      *reinterpret_cast<__nv_bfloat162*>(Qs + r * LDE + c) = __floats2bfloat162_rn(v.x, v.y);
      *reinterpret_cast<__nv_bfloat162*>(Qs + r * LDE + c + 2) = __floats2bfloat162_rn(v.z, v.w);
    }
  }
  if (tid < R) { Ms[tid] = -FLT_MAX; Ls[tid] = 0.f; As[tid] = 1.f; }
  float acc[MB][kMaxPairs][2][4];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int i = 0; i < kMaxPairs; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[mb][i][j][k] = 0.f;
  const int npairs = C / 16;
  const int g = lane >> 2, t4 = lane & 3;
  const int smb = w & 3, skh = w >> 2;   // scores: this warp's row block and key half
  const float scale_log2 = a.scale * 1.4426950408889634f;

  // Two barriers per tile.  One group is committed per tile (an empty one past the end), so waiting for all but the newest
  // NST - 2 means: the next tile to be read has landed.  Tile ti + NST - 1 is fetched after the barrier behind the scores of
  // tile ti, into the buffer that the values of tile ti - 1 read; the wait for tile ti + 1 stands before the barrier
  // between softmax and values, which therefore also publishes that tile to every warp.
  if (NST == 3) cp_async_wait_group<1>(); else cp_async_wait_group<0>();
  __syncthreads();
  int buf = 0;   // ti % NST
  for (int ti = 0; ti < ntiles; ++ti) {
    const bf16* Kt = Ks + static_cast<size_t>(buf) * KT * LDE;
    const int nb = buf == 0 ? NST - 1 : buf - 1;
    buf = buf + 1 == NST ? 0 : buf + 1;
    // ---- scores: 16 rows x 16 keys per warp
    {
      float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f}, d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t qa = smem_addr(Qs + (smb * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDE + 8 * (lane >> 4));
      const uint32_t ka = smem_addr(Kt + (skh * 16 + (lane & 7) + 8 * (lane >> 4)) * LDE + 8 * ((lane >> 3) & 1));
      // E is a multiple of 16: pairs of k-steps with all four fragment loads ahead of the four mma, then an odd last one
      int ks = 0;
#pragma unroll 2
      for (; ks + 32 <= E; ks += 32) {
        uint32_t af[4], bf[4], ag[4], bg[4];
        ldsm_x4(af, qa + ks * 2);
        ldsm_x4(bf, ka + ks * 2);     // keys 0-7: k lo, k hi; keys 8-15: k lo, k hi
        ldsm_x4(ag, qa + (ks + 16) * 2);
        ldsm_x4(bg, ka + (ks + 16) * 2);
        mma16816(c0, af, bf[0], bf[1]);
        mma16816(c1, af, bf[2], bf[3]);
        mma16816(d0, ag, bg[0], bg[1]);
        mma16816(d1, ag, bg[2], bg[3]);
      }
      if (ks < E) {
        uint32_t af[4], bf[4];
        ldsm_x4(af, qa + ks * 2);
        ldsm_x4(bf, ka + ks * 2);
        mma16816(c0, af, bf[0], bf[1]);
        mma16816(c1, af, bf[2], bf[3]);
      }
      float* sp = Ss + (smb * 16 + g) * LDS + skh * 16 + 2 * t4;
      sp[0] = c0[0] + d0[0]; sp[1] = c0[1] + d0[1];
      sp[8 * LDS] = c0[2] + d0[2]; sp[8 * LDS + 1] = c0[3] + d0[3];
      sp[8] = c1[0] + d1[0]; sp[9] = c1[1] + d1[1];
      sp[8 * LDS + 8] = c1[2] + d1[2]; sp[8 * LDS + 9] = c1[3] + d1[3];
    }
    __syncthreads();
    if (ti + NST - 1 < ntiles) load_tile(ti + NST - 1, nb);
    cp_async_commit();
    // ---- online softmax: thread -> (row, 8 keys); scores in units of log 2 so that the exponentials are single ex2
    {
      const int srow = tid >> 2, sk = (tid & 3) * 8;
      const int s_tq = srow / HB;
      const bool s_valid = s_tq < ntq && h0 + srow % HB < a.heads;
      const int s_pos = p_first + s_tq;
      const int j0 = lo + ti * KT + sk;
      float sv[8], mx = -FLT_MAX;
      const float4 x0 = *reinterpret_cast<const float4*>(Ss + srow * LDS + sk);
      const float4 x1 = *reinterpret_cast<const float4*>(Ss + srow * LDS + sk + 4);
      const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int j = j0 + i;
        const bool vis = s_valid && j <= s_pos && j > s_pos - a.window;
        sv[i] = vis ? xs[i] * scale_log2 : -FLT_MAX;
        mx = fmaxf(mx, sv[i]);
      }
      const float m_old = Ms[srow];
      for (int o = 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      // the reference point of the exponentials follows the maximum only when that has grown by more than kLazyMax: terms
      // stay below 2^kLazyMax, the final division cancels the reference point, and most tiles leave the accumulators alone
      constexpr float kLazyMax = 8.f;
      const float m_new = (m_old == -FLT_MAX || mx > m_old + kLazyMax) ? fmaxf(m_old, mx) : m_old;
      float sum = 0.f;
      float pv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) { pv[i] = sv[i] == -FLT_MAX ? 0.f : exp2f(sv[i] - m_new); sum += pv[i]; }
      for (int o = 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
      for (int i = 0; i < 8; i += 2) *reinterpret_cast<__nv_bfloat162*>(Ps + srow * LDP + sk + i) = __floats2bfloat162_rn(pv[i], pv[i + 1]);
      __syncwarp();
      if ((tid & 3) == 0) {
        const float al = m_old == -FLT_MAX ? 0.f : exp2f(m_old - m_new);
        Ms[srow] = m_new;
        Ls[srow] = Ls[srow] * al + sum;
        As[srow] = m_new == -FLT_MAX ? 1.f : al;
      }
    }
    if (NST == 3) cp_async_wait_group<1>(); else cp_async_wait_group<0>();
    __syncthreads();
    // ---- values: this warp's column pairs, for every row block
    {
      uint32_t pa[MB][2][4];
      float al0[MB], al1[MB];
      const uint32_t pbase = smem_addr(Ps + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LDP + 8 * (lane >> 4));
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        al0[mb] = As[mb * 16 + g];
        al1[mb] = As[mb * 16 + g + 8];
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) ldsm_x4(pa[mb][ks], pbase + (mb * 16 * LDP + ks * 16) * 2);
      }
      // after the first tiles a row's maximum seldom moves: the accumulators are rescaled only when some factor is not 1
      bool moved = false;
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) moved = moved || al0[mb] != 1.f || al1[mb] != 1.f;
      moved = __any_sync(0xffffffffu, moved);
#pragma unroll
      for (int i = 0; i < kMaxPairs; ++i) {
        const int pp = w + 8 * i;
        if (pp < npairs) {
          if (moved) {
#pragma unroll
            for (int mb = 0; mb < MB; ++mb)
#pragma unroll
              for (int j = 0; j < 2; ++j) { acc[mb][i][j][0] *= al0[mb]; acc[mb][i][j][1] *= al0[mb]; acc[mb][i][j][2] *= al1[mb]; acc[mb][i][j][3] *= al1[mb]; }
          }
          const uint32_t vb = smem_addr(Kt + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LDE + 16 * pp + 8 * (lane >> 4));
#pragma unroll
          for (int ks = 0; ks < 2; ++ks) {
            uint32_t bv[4];
            ldsm_x4_trans(bv, vb + ks * 16 * LDE * 2);
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
              mma16816(acc[mb][i][0], pa[mb][ks], bv[0], bv[1]);
              mma16816(acc[mb][i][1], pa[mb][ks], bv[2], bv[3]);
            }
          }
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = mb * 16 + g + 8 * half, tq = r / HB, h = h0 + r % HB;
      if (tq >= ntq || h >= a.heads) continue;
      const float inv = 1.0f / Ls[r];
      float* out = a.olat + (static_cast<long long>(tok0 + tq0 + tq) * a.heads + h) * C;
#pragma unroll
      for (int i = 0; i < kMaxPairs; ++i) {
        const int pp = w + 8 * i;
        if (pp < npairs) {
#pragma unroll
          for (int j = 0; j < 2; ++j)
            *reinterpret_cast<float2*>(out + 16 * pp + 8 * j + 2 * t4) = make_float2(acc[mb][i][j][2 * half] * inv, acc[mb][i][j][2 * half + 1] * inv);
        }
      }
    }
}

size_t latent_mma_wide_smem(int E, int stages) {
  const size_t LDE = E + 8, R = kWideRows, KT = kWideKeys;
  return (R * LDE + stages * KT * LDE) * 2 + R * (KT + 4) * 4 + R * (KT + 8) * 2 + 3 * R * 4;
}

size_t latent_mma_smem(int E, int MB) {
  const size_t LDE = E + 8, R = 16 * MB;
  return (R * LDE + 2 * kKeys * LDE) * 2 + R * (kKeys + 4) * 4 + R * (kKeys + 8) * 2 + 3 * R * 4;
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
  // bf16 caches whose widths fit the fragments run on the tensor cores (B200_NX_ATTN_MMA=0: A/B knob)
  const int E = a.kv_rank + a.rot_dim;
  const char* ev = getenv("B200_NX_ATTN_MMA");
  if (a.t == DT_BF16 && a.seqs && E % 16 == 0 && a.kv_rank % 16 == 0 && a.kv_rank <= 8 * kMaxPairs * 16 && latent_mma_smem(E, 1) <= 220 * 1024 &&
      !(ev && atoi(ev) == 0)) {
    // once per device, for the largest tile the dispatch admits: the attribute is a limit, not a per-launch size
    static std::atomic<unsigned long long> attr1{0}, attr2{0};
    const int HB = a.heads < 16 ? a.heads : 16;
    // two row blocks when the step is mostly prompt portions and 32 rows still hold whole tokens
    const bool two = a.T >= 2 * a.nseq && 32 / HB >= 2 && latent_mma_smem(E, 2) <= 220 * 1024;
    const int TQ = (two ? 32 : 16) / HB;
    // few CTAs and long windows (decode of a handful of sequences): split every window over several CTAs and merge
    int sms = 148;
    { int dev = 0; if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
    const int ctas = ((a.T + TQ - 1) / TQ) * ((a.heads + HB - 1) / HB);
    const int key_tiles = (std::min(a.window, std::max(a.max_ctx, 1)) + kKeys - 1) / kKeys;
    int nsplit = 1;
    const char* se = getenv("B200_NX_ATTN_SPLIT");   // A/B knob: 1 = never split
    if (a.split_ws && ctas * 2 <= sms && key_tiles >= 4) nsplit = std::min(std::min(sms / ctas, key_tiles / 2), 16);
    if (se) nsplit = std::max(1, std::min(atoi(se), 16));
    if (nsplit > 1 && (!a.split_ws || static_cast<long long>(a.T) * a.heads * nsplit * (a.kv_rank + 2) > a.split_ws_floats)) nsplit = 1;
    // steps of long prompt portions with CTAs enough for every SM: 64 rows per CTA (B200_NX_ATTN_WIDE=1 forces, 0 forbids)
    const int TQW = kWideRows / HB;
    const char* we = getenv("B200_NX_ATTN_WIDE");
    bool wide = two && a.T >= 4 * a.nseq && ((a.T + TQW - 1) / TQW) * ((a.heads + HB - 1) / HB) >= sms;
    if (we) wide = two && atoi(we) != 0;
    // three key buffers: every latent width whose 32-row form fits shared memory also fits them
    constexpr int stages = 3;
    if (wide && latent_mma_wide_smem(E, stages) <= 220 * 1024 && !se) {
      static std::atomic<unsigned long long> attrw{0};
      if (!ensure_dynamic_smem(latent_attn_mma_wide_kernel, 220 * 1024, &attrw)) return -2;
      dim3 gridw((a.T + TQW - 1) / TQW + a.nseq, (a.heads + HB - 1) / HB);
      latent_attn_mma_wide_kernel<<<gridw, 256, latent_mma_wide_smem(E, stages), st>>>(a, a.seqs, a.nseq, TQW, HB, stages);
      return cudaGetLastError() == cudaSuccess ? 0 : -2;
    }
    dim3 grid((a.T + TQ - 1) / TQ + a.nseq, (a.heads + HB - 1) / HB, nsplit);
    if (two) {
      if (!ensure_dynamic_smem(latent_attn_mma_kernel<2>, 220 * 1024, &attr2)) return -2;
      latent_attn_mma_kernel<2><<<grid, 256, latent_mma_smem(E, 2), st>>>(a, a.seqs, a.nseq, TQ, HB, nsplit, a.split_ws);
    } else {
      if (!ensure_dynamic_smem(latent_attn_mma_kernel<1>, 220 * 1024, &attr1)) return -2;
      latent_attn_mma_kernel<1><<<grid, 256, latent_mma_smem(E, 1), st>>>(a, a.seqs, a.nseq, TQ, HB, nsplit, a.split_ws);
    }
    if (cudaGetLastError() != cudaSuccess) return -2;
    if (nsplit > 1) {
      const long long rows = static_cast<long long>(a.T) * a.heads;
      latent_attn_merge_kernel<<<static_cast<unsigned>((rows + 3) / 4), 128, 0, st>>>(a.split_ws, a.olat, a.kv_rank, nsplit, rows);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
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
