// Host launchers of the kernels behind the non-Llama model designs: a shape-agnostic linear layer (plain, batched per
// head, or grouped per expert), Dynamic-Tanh norm fused with the fp32 residual update, a hashed bigram embedding,
// gated linear attention (decayed outer-product state per sequence slot), latent attention (paged low-rank KV with a
// shared rotated key and a sliding window), group-limited expert routing, and the gated activations they use.
//
// Storage type: every activation / weight matrix is either bf16 or fp32 (DType); the residual stream, recurrent
// states, router scores, decays, softmax and norm statistics are always fp32.  All pointers are device pointers.
// Launchers return 0 on success and a negative number on a bad shape or a launch error.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace b200 {

enum DType { DT_BF16 = 0, DT_F32 = 1 };
inline size_t dtype_bytes(DType t) { return t == DT_BF16 ? 2 : 4; }

// ---------------------------------------------------------------- linear (linear.cu)
enum LinearAct { LIN_NONE = 0, LIN_RELU2 = 1 };   // epilogue on the fp32 accumulator: identity, max(y, 0)^2
// Y[b][t, n] = act( sum_k X[b][row(t), k] * W[b'][n, k] ),  t < T, n < N.
//   batch > 1: X, W, Y advance by xbs / wbs / ybs elements per batch index (per-head projections inside wider rows).
//   x_rows (optional): row(t) = x_rows[t], a negative entry reads a zero row and its output row is not written.
//   tile_group (optional, needs T % 64 == 0 capacity): rows [64 i, 64 i + 64) use weight matrix W + tile_group[i] * wbs;
//     a negative entry skips the tile (expert-grouped rows padded to the tile size).
// The accumulation order of one output element never depends on T or on the other rows (k ascending inside a tile
// kernel, a fixed lane pattern in the few-row kernel), so a row's result does not depend on what shares the batch.
struct LinearArgs {
  const void* X; const void* W; void* Y;
  DType tx, tw, ty;
  int T, N, K;
  int ldx, ldw, ldy;
  int batch; long long xbs, wbs, ybs;
  const int* x_rows;
  const int* tile_group;
  int act;
};
inline LinearArgs linear_args(const void* X, DType tx, const void* W, DType tw, void* Y, DType ty, int T, int N, int K) {
  LinearArgs a = {X, W, Y, tx, tw, ty, T, N, K, K, K, N, 1, 0, 0, 0, nullptr, nullptr, LIN_NONE};
  return a;
}
int linear(const LinearArgs& a, cudaStream_t st);
// `rows` rows (a handful: the expert choices of a decode step), row r reading X row src_rows[r] (or r / src_div), writing Y row
// dst_rows[r], with weight matrix W + groups[r] * wbs; a.T, a.batch, x_rows and tile_group are not used.
struct PickedRows {
  int rows;
  const int* src_rows; int src_div;
  const int* dst_rows;
  const int* groups;
};
int linear_picked_rows(const LinearArgs& a, const PickedRows& p, cudaStream_t st);

// ---------------------------------------------------------------- embedding, norm, activations (norm_act.cu)
// x[t] = embed[ids[t]] + bigram[row], row = (prev * mul_prev + id * mul_cur) mod buckets, or row `buckets` when
// prev_ids[t] < 0 (the first token of a sequence).  x is fp32 [T, W]; tables are [*, W] of type tw.
int embed_bigram(const void* embed, const void* bigram, DType tw, const int* ids, const int* prev_ids, float* x, int T, int W,
                 int vocab, int buckets, long long mul_prev, long long mul_cur, cudaStream_t st);
// Dynamic Tanh with the residual update in front of it.  For r < rows, t = row_index ? row_index[r] : r:
//   if (a || f) x[t] += mult * (a[t] + f[t])   (fp32, in place; a, f of type ta, either may be null)
//   if (y)      y[r] = tanh(alpha[0] * x[t]) * w + b          (w, b, alpha fp32; y of type ty)
int residual_dyt(float* x, const void* a, const void* f, DType ta, float mult, const float* w, const float* b, const float* alpha,
                 void* y, DType ty, const int* row_index, int rows, int W, cudaStream_t st);
// Clamped gated unit: row t of gu (leading dimension ldgu) holds gate [F] | up [F]; g = min(gate, limit), u = clamp(up, -limit, limit),
// y = g * sigmoid(slope * g) * (u + 1)
int glu_clamped(const void* gu, int ldgu, void* y, int ldy, DType t, int T, int F, float limit, float slope, cudaStream_t st);
// y[t, i] *= sigmoid(g[t, i]), i < n (leading dimensions ldy, ldg)
int sigmoid_gate(void* y, int ldy, const void* g, int ldg, DType t, int T, int n, cudaStream_t st);
// p[i] = offset + scale * u_i, u uniform in [-1, 1) from a counter hash of (seed, i): seeded random weights for benchmarks
int fill_uniform(void* p, DType t, size_t n, uint64_t seed, float scale, float offset, cudaStream_t st);
int argmax_f32(const float* logits, int* out, int S, int V, cudaStream_t st);

// ---------------------------------------------------------------- gated linear attention (gla.cu)
// Per sequence and head: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T (q_t * q_scale), alpha = sigmoid(z + z_bias)^(inv_tau),
// all in fp32.  q, k, v are column blocks of one row-major buffer (leading dimension ld, column offsets q_off / k_off /
// v_off; heads x dim, heads x dim, heads x vdim).  z: fp32 [T, heads * dim] pre-activations, replaced by the decays.  states: fp32 [slot][heads][dim][vdim].
// seqs: int [nseq][8] = {first row, rows, first position, state slot, ...}; a sequence whose first position is 0 starts
// from a zero state whatever its slot held.  o: fp32 [T, heads * vdim].
struct GlaArgs {
  const void* qkv; DType t; int ld, q_off, k_off, v_off;
  float* z; const float* z_bias; float inv_tau, q_scale;   // z is overwritten with the decays
  int T;                                                      // rows of z (tokens in the step)
  float* states; const int* seqs; int nseq;
  int heads, dim, vdim;
  float* o;
};
int gla_scan(const GlaArgs& a, cudaStream_t st);
// y[t, h * vdim + :] (leading dimension ldy) = o[t, h, :] / sqrt(mean(o^2) + eps) * w * silu(g[t, h, :])   (w: fp32 [vdim], shared by the heads)
int gla_out_gate(const float* o, const void* g, int ldg, const float* w, float eps, void* y, int ldy, DType t, int T, int heads, int vdim,
                 cudaStream_t st);

// ---------------------------------------------------------------- latent attention (latent_attention.cu)
// Rotation table for interleaved pairs (2i, 2i+1): cs[p][i] = (cos, sin)(p * base^(-2i/dims)), computed in double.
int rope_table_interleaved(float2* table, int max_pos, int dims, double base, cudaStream_t st);
// Per token: the first kv_rank columns of dkv are unit-RMS-normed (eps inside the root) and scaled by norm_w -> cache row,
// the next rot_dim columns are rotated (first rot_dims of them) -> cache row tail; the rotated part of every query head
// (q laid out [heads][dim + rot_dim]) is rotated into qlat[t][h][kv_rank ...] (fp32, row stride heads * (kv_rank + rot_dim)).
// cache: [slot][kv_rank + rot_dim] of type t, slot = page * page_size + offset as given by slots[t].
struct LatentPrepArgs {
  const void* q; int ldq; const void* dkv; int lddkv; DType t;
  const float* norm_w; float eps;
  const float2* rope; int rot_dims;
  const int* positions; const int* slots;
  void* cache; float* qlat;
  int T, heads, dim, rot_dim, kv_rank;
};
int latent_prep(const LatentPrepArgs& a, cudaStream_t st);
// Sliding-window softmax attention in latent space: for token t at position p of sequence s, keys j with
// max(0, p - window + 1) <= j <= p; score = qlat[t, h] . cache[j] * scale; olat[t, h] = sum_j softmax_j * cache[j][:kv_rank].
struct LatentAttnArgs {
  const float* qlat; const void* cache; DType t;
  const int* positions; const int* seq_of_tok; const int* block_tables; int max_blocks, page;
  float* olat;
  int T, heads, kv_rank, rot_dim, window; float scale;
  const int* seqs; int nseq;   // the step's per-sequence table ({first row, rows, first position, ...}); needed by the tensor-core kernel
  int max_ctx;                 // longest context (position of a last token + 1) in the step, for the split decision
  float* split_ws; long long split_ws_floats;   // optional workspace of the split form: [rows][splits][kv_rank + 2] fp32
};
int latent_attention(const LatentAttnArgs& a, cudaStream_t st);

// ---------------------------------------------------------------- mixture of experts (moe.cu)
// scores: fp32 [T, E] router logits in, clobbered.  softmax over E; experts form `groups` equal groups of neighbours, a
// group's score is its largest member, only the `keep` best groups are eligible; the `top` largest eligible scores are
// chosen (ties: lower index) and used unchanged as weights.  topk_ids / topk_w: [T, top].
int moe_route(float* scores, int* topk_ids, float* topk_w, int T, int E, int groups, int keep, int top, cudaStream_t st);
// Sort the T * top (token, choice) pairs by expert into 64-row tiles: sorted_rows[cap] = token of each sorted row or -1,
// tile_group[cap / 64] = expert of each tile or -1, pair_pos[T * top] = sorted row of each pair.  cap >= T*top + E*64.
// expert_rows (optional): [E][2] = {first sorted row, rows} of every expert.
int moe_align(const int* topk_ids, int T, int top, int E, int* sorted_rows, int* tile_group, int* pair_pos, int cap, cudaStream_t st,
              int* expert_rows = nullptr);
// out[t] = sum_k topk_w[t, k] * y[pair_pos[t * top + k]]   (y [cap, W] fp32 or bf16, k ascending)
int moe_combine(const void* y, DType ty, const int* pair_pos, const float* topk_w, void* out, DType t, int T, int top, int W, cudaStream_t st);
// bf16 helpers of the per-expert tensor-core path: x rows in sorted order (negative source row -> zeros), max(p, 0)^2 in place
int moe_gather_bf16(const void* x, const int* sorted_rows, void* out, int rows, int W, cudaStream_t st);
int relu2_bf16(void* p, long long n, cudaStream_t st);

}  // namespace b200
