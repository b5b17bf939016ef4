// Nomanex: a decoder-only design of parallel layers on an fp32 residual stream.
//
//   x_0[t]   = embed[token] + bigram[hash(previous token, token)]
//   h        = dyt(x) = tanh(alpha x) w + b                         (Dynamic Tanh: no statistics)
//   x       <- x + m (mixer(h) + ff(h))                             (one norm, both sublayers read it)
//   mixer    = gated linear attention (gla.cu) | latent attention with a sliding window (latent_attention.cu)
//   ff       = clamped gated unit | group-limited mixture of squared-ReLU experts (moe.cu) | none
//   logits   = head dyt_final(x)
// A layer may name another layer whose weights it uses (`weights_of`); it keeps a cache / state of its own.
//
// Per layer the kernel sequence is: ONE input projection for everything that reads h (mixer projections, the decay's
// low-rank input, the dense unit's gate and up rows are concatenated row-wise at load), the mixer's own kernels, ONE
// output projection over the concatenated [mixer output | ff hidden] columns (W_o and W_down concatenated column-wise,
// so the sum mixer(h) + ff(h) comes out of the accumulator), and the residual update fused with the next layer's norm.
// Every size and constant comes from config.json; the storage type of matrices and activations is bf16 or fp32, with
// the residual, states, router, decays, softmax and norms in fp32 either way.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <string.h>

#include <algorithm>

#include "errors.h"
#include "gemm.h"
#include "model.h"

namespace b200 {
namespace {

typedef __nv_bfloat16 bf16;

enum { MIX_GLA = 0, MIX_LATENT = 1 };
enum { FF_NONE = 0, FF_DENSE = 1, FF_MOE = 2 };

struct LayerSpec {
  int mixer = MIX_GLA, ff_kind = FF_NONE;
  int weights_of = -1;   // index of the layer that owns the weights (itself when it has its own)
  // mixer
  int heads = 0, dim = 0, vdim = 0;
  float tau = 1.f;                                 // gla
  int a_rank = 0;                                  // gla: rows of the decay's first projection (from the tensor)
  int kv_rank = 0, rot_dim = 0, rot_dims = 0, window = 0;   // latent attention
  double rot_base = 10000.0;
  float scale = 1.f;
  // feed-forward
  int ff = 0;
  float limit = 0.f;
  int experts = 0, top = 0, groups = 1, keep = 1;
  // derived column layout of the input projection's output row
  int n_in = 0, off_q = 0, off_k = 0, off_v = 0, off_g = 0, off_a1 = 0, off_dkv = 0, off_gu = 0;
  int k_out = 0;   // columns of the output projection's input: heads * vdim (+ ff for a dense unit)
};

struct LayerWeights {
  void* w_in = nullptr;    // [n_in, width]
  void* w_out = nullptr;   // [width, k_out]
  float *norm_w = nullptr, *norm_b = nullptr, *norm_alpha = nullptr;
  // gla
  void* a2 = nullptr;      // [heads * dim, a_rank]
  float *a2_b = nullptr, *o_norm = nullptr;
  // latent attention
  float* c_norm = nullptr;
  void* uk_t = nullptr;    // [heads][kv_rank][dim]: W_uk transposed per head (the latent query projection)
  void* uv = nullptr;      // [heads * vdim, kv_rank]
  float2* rope = nullptr;  // [max_model_len][rot_dims / 2]
  // moe
  void* router = nullptr;  // [experts, width]
  void* e_up = nullptr;    // [experts][ff][width]
  void* e_down = nullptr;  // [experts][width][ff]
  GemmPlan p_in, p_out;    // tcgen05 projections (bf16 storage, K % 8 == 0)
  std::vector<GemmPlan> p_eup, p_edown;   // per expert, for steps large enough to pay for a count read-back
  CUtensorMap xm_out[kGemmNumBlockN];   // activation maps over the output projection's input [Tcap, k_out]
  bool tc_in = false, tc_out = false;
};

struct LayerRun {
  void* cache = nullptr;    // latent: [num_blocks * page][kv_rank + rot_dim]
  float* state = nullptr;   // gla: [slots][heads][dim][vdim]
};

bool jnum(const JVal* o, const char* k, double* out) {
  const JVal* v = o ? o->get(k) : nullptr;
  if (!v || v->type != JVal::Num) return false;
  *out = v->num;
  return true;
}

class Nomanex : public Model {
 public:
  DType dt;
  int V = 0, W = 0;
  float eps = 1e-5f, mult = 1.f;
  int buckets = 1;
  long long mul_prev = 0, mul_cur = 0;
  std::vector<LayerSpec> spec;
  std::vector<LayerWeights> wts;   // indexed like spec; only owners are filled
  std::vector<LayerRun> run;
  ModelEnv env;
  // weights outside the layers
  void *embed = nullptr, *bigram = nullptr, *head = nullptr;
  float *fin_w = nullptr, *fin_b = nullptr, *fin_alpha = nullptr;
  // activations
  float* x = nullptr;
  void *h = nullptr, *inb = nullptr, *ycat = nullptr, *ao = nullptr, *fo = nullptr, *hrow = nullptr, *eact = nullptr;
  float *z = nullptr, *o32 = nullptr, *qlat = nullptr, *olat = nullptr, *scores = nullptr, *topw = nullptr, *edown = nullptr,
        *logits = nullptr;
  int *topi = nullptr, *sorted_rows = nullptr, *tile_group = nullptr, *pair_pos = nullptr;
  int row_cap = 0, moe_cap = 0;
  float* split_ws = nullptr;       // partials of the split attention form (decode of a few long sequences)
  long long split_ws_floats = 0;
  void *hsorted = nullptr, *edown16 = nullptr;   // per-expert tensor-core path: gathered inputs, bf16 expert outputs
  int *expert_rows = nullptr, *expert_rows_host = nullptr;
  std::vector<void*> allocs;
  // tcgen05 projections
  float* gemm_ws = nullptr;
  int* gemm_counters = nullptr;
  CUtensorMap xm_h[kGemmNumBlockN];
  bool use_tc = false;

  explicit Nomanex(DType d) : dt(d) {}
  ~Nomanex() override {
    for (auto& w : wts) {
      if (w.tc_in) gemm_plan_destroy(&w.p_in);
      if (w.tc_out) gemm_plan_destroy(&w.p_out);
    }
    if (expert_rows_host) cudaFreeHost(expert_rows_host);
    for (void* p : allocs) cudaFree(p);
  }
  // (profiling events are released with the context)
  const char* arch() const override { return "Nomanex"; }
  int vocab() const override { return V; }

  size_t cache_bytes_per_block(int page) const override {
    size_t b = 0;
    for (auto& s : spec)
      if (s.mixer == MIX_LATENT) b += static_cast<size_t>(page) * (s.kv_rank + s.rot_dim) * dtype_bytes(dt);
    return b;
  }
  int cache_window() const override {
    int w = 0;
    for (auto& s : spec)
      if (s.mixer == MIX_LATENT) {
        if (s.window >= (1 << 30)) return 0;
        w = std::max(w, s.window);
      }
    return w;
  }
  size_t state_bytes_per_slot() const override {
    size_t b = 0;
    for (auto& s : spec)
      if (s.mixer == MIX_GLA) b += static_cast<size_t>(s.heads) * s.dim * s.vdim * sizeof(float);
    return b;
  }

  // ------------------------------------------------------------ config.json
  bool parse(const JVal& c, std::string* err) {
    double d = 0;
    if (!jnum(&c, "vocab", &d) || d < 1) { *err = "config: vocab"; return false; }
    V = static_cast<int>(d);
    if (!jnum(&c, "width", &d) || d < 1) { *err = "config: width"; return false; }
    W = static_cast<int>(d);
    if (jnum(&c, "residual_mult", &d)) mult = static_cast<float>(d);
    if (jnum(c.get("norm"), "eps", &d)) eps = static_cast<float>(d);
    const JVal* em = c.get("embedding");
    const JVal* bg = em ? em->get("bigram") : nullptr;
    if (!bg) { *err = "config: embedding.bigram"; return false; }
    if (!jnum(bg, "buckets", &d) || d < 1) { *err = "config: bigram.buckets"; return false; }
    buckets = static_cast<int>(d);
    if (jnum(bg, "mul_prev", &d)) mul_prev = static_cast<long long>(d);
    if (jnum(bg, "mul_cur", &d)) mul_cur = static_cast<long long>(d);
    const JVal* ls = c.get("layers");
    if (!ls || ls->type != JVal::Arr || ls->arr.empty()) { *err = "config: layers"; return false; }
    for (size_t i = 0; i < ls->arr.size(); ++i) {
      const JVal& L = ls->arr[i];
      LayerSpec s;
      const JVal* ty = L.get("type");
      if (!ty || ty->type != JVal::Str) { *err = "config: layer type"; return false; }
      if (ty->str == "gla") s.mixer = MIX_GLA;
      else if (ty->str == "latent_attention") s.mixer = MIX_LATENT;
      else { *err = "config: unknown mixer \"" + ty->str + "\""; return false; }
      const JVal* mx = L.get("mixer");
      if (!mx || mx->type != JVal::Obj) { *err = "config: layer mixer"; return false; }
      auto need = [&](const JVal* o, const char* k, int* out) {
        double v = 0;
        if (!jnum(o, k, &v) || v < 1 || v != floor(v)) { *err = std::string("config: layer ") + std::to_string(i) + " " + k; return false; }
        *out = static_cast<int>(v);
        return true;
      };
      if (!need(mx, "heads", &s.heads) || !need(mx, "dim", &s.dim) || !need(mx, "vdim", &s.vdim)) return false;
      if (s.mixer == MIX_GLA) {
        if (!jnum(mx, "tau", &d) || !(d > 0)) { *err = "config: gla tau"; return false; }
        s.tau = static_cast<float>(d);
      } else {
        if (!need(mx, "kv_rank", &s.kv_rank) || !need(mx, "rot_dim", &s.rot_dim)) return false;
        const JVal* rot = mx->get("rot");
        s.rot_dims = s.rot_dim;
        if (jnum(rot, "dims", &d)) s.rot_dims = static_cast<int>(d);
        if (jnum(rot, "base", &d)) s.rot_base = d;
        if (s.rot_dims < 0 || s.rot_dims > s.rot_dim || s.rot_dims % 2) { *err = "config: rot.dims"; return false; }
        s.window = 1 << 30;   // no mask entry: full causal attention
        if (const JVal* mk = mx->get("mask")) if (jnum(mk, "size", &d) && d >= 1) s.window = static_cast<int>(std::min(d, 1073741824.0));
        s.scale = 1.0f / sqrtf(static_cast<float>(s.dim + s.rot_dim));
        if (jnum(mx, "scale", &d)) s.scale = static_cast<float>(d);
      }
      const JVal* mlp = L.get("mlp");
      if (mlp && mlp->type == JVal::Obj) {
        const JVal* kind = mlp->get("kind");
        if (!kind || kind->type != JVal::Str) { *err = "config: mlp.kind"; return false; }
        if (kind->str == "dense") {
          s.ff_kind = FF_DENSE;
          if (!need(mlp, "ff", &s.ff)) return false;
          if (!jnum(mlp, "limit", &d)) { *err = "config: mlp.limit"; return false; }
          s.limit = static_cast<float>(d);
        } else if (kind->str == "moe") {
          s.ff_kind = FF_MOE;
          const JVal* ex = mlp->get("expert");
          const JVal* rt = mlp->get("router");
          if (!need(ex, "ff", &s.ff) || !need(rt, "experts", &s.experts) || !need(rt, "top", &s.top)) return false;
          s.groups = 1; s.keep = 1;
          if (const JVal* g = rt ? rt->get("groups") : nullptr) {
            if (!need(g, "count", &s.groups) || !need(g, "keep", &s.keep)) return false;
          }
          if (s.experts % s.groups || s.groups > 64 || s.keep > s.groups || s.top > s.keep * (s.experts / s.groups)) { *err = "config: router groups"; return false; }
        } else { *err = "config: unknown mlp kind \"" + kind->str + "\""; return false; }
      }
      s.weights_of = static_cast<int>(i);
      if (jnum(&L, "weights_of", &d)) {
        if (d < 0 || d >= static_cast<double>(ls->arr.size()) || d != floor(d)) { *err = "config: weights_of out of range"; return false; }
        s.weights_of = static_cast<int>(d);
      }
      spec.push_back(s);
    }
    // a layer without tensors of its own follows `weights_of` to the layer that has them
    for (size_t i = 0; i < spec.size(); ++i) {
      int j = spec[i].weights_of;
      for (size_t hops = 0; spec[j].weights_of != j; ++hops) {
        if (hops > spec.size()) { *err = "config: weights_of forms a cycle"; return false; }
        j = spec[j].weights_of;
      }
      spec[i].weights_of = j;
      const LayerSpec &o = spec[j], &s = spec[i];
      if (o.mixer != s.mixer || o.heads != s.heads || o.dim != s.dim || o.vdim != s.vdim || o.ff_kind != s.ff_kind || o.ff != s.ff ||
          o.kv_rank != s.kv_rank || o.rot_dim != s.rot_dim || o.experts != s.experts) { *err = "config: a layer sharing weights must have the owner's sizes"; return false; }
    }
    return true;
  }

  // column layout of the input projection (needs a_rank, known once the checkpoint or the default is seen)
  void layout(LayerSpec& s) {
    int at = 0;
    if (s.mixer == MIX_GLA) {
      s.off_q = at; at += s.heads * s.dim;
      s.off_k = at; at += s.heads * s.dim;
      s.off_v = at; at += s.heads * s.vdim;
      s.off_g = at; at += s.heads * s.vdim;
      s.off_a1 = at; at += s.a_rank;
    } else {
      s.off_q = at; at += s.heads * (s.dim + s.rot_dim);
      s.off_dkv = at; at += s.kv_rank + s.rot_dim;
      s.off_g = at; at += s.heads * s.vdim;
    }
    at = (at + 7) / 8 * 8;   // keeps the dense unit's columns 16-byte aligned
    if (s.ff_kind == FF_DENSE) { s.off_gu = at; at += 2 * s.ff; }
    s.n_in = (at + 7) / 8 * 8;
    s.k_out = s.heads * s.vdim + (s.ff_kind == FF_DENSE ? s.ff : 0);
  }

  template <typename P>
  int dalloc(P** p, size_t bytes) {
    void* q = nullptr;
    if (cudaMalloc(&q, std::max<size_t>(bytes, 16)) != cudaSuccess) { set_error("Nomanex: device allocation of %zu bytes failed", bytes); return -3; }
    cudaMemsetAsync(q, 0, std::max<size_t>(bytes, 16), env.stream);
    allocs.push_back(q);
    *p = static_cast<P*>(q);
    return 0;
  }

  // The rank of the decay's low-rank projection is a tensor shape, not a config entry: it is read from the checkpoint
  // before init() sizes the buffers (16 when the weights are random).
  int inspect(const CheckpointReader& ck, std::string* err) override {
    for (size_t i = 0; i < spec.size(); ++i) {
      if (spec[i].mixer != MIX_GLA) continue;
      std::vector<int64_t> sh;
      const std::string name = "l" + std::to_string(spec[i].weights_of) + ".mix.a1";
      if (!ck.shape(name, &sh) || sh.size() != 2 || sh[0] < 1) { *err = "missing or malformed tensor " + name; return -4; }
      spec[i].a_rank = static_cast<int>(sh[0]);
    }
    return 0;
  }

  int init(const ModelEnv& e) override {
    env = e;
    const size_t es = dtype_bytes(dt);
    wts.resize(spec.size());
    run.resize(spec.size());
    int max_in = 8, max_kout = 8, max_hd = 1, max_hv = 1, max_ql = 1, max_ol = 1, max_e = 1, max_top = 1, max_eff = 1;
    bool any_moe = false;
    for (auto& s : spec) {
      if (s.mixer == MIX_GLA && s.a_rank == 0) s.a_rank = 16;
      layout(s);
      max_in = std::max(max_in, s.n_in);
      max_kout = std::max(max_kout, s.k_out);
      max_hd = std::max(max_hd, s.heads * s.dim);
      max_hv = std::max(max_hv, s.heads * s.vdim);
      if (s.mixer == MIX_LATENT) {
        max_ql = std::max(max_ql, s.heads * (s.kv_rank + s.rot_dim));
        max_ol = std::max(max_ol, s.heads * s.kv_rank);
      }
      if (s.ff_kind == FF_MOE) {
        any_moe = true;
        max_e = std::max(max_e, s.experts);
        max_top = std::max(max_top, s.top);
        max_eff = std::max(max_eff, s.ff);
      }
    }
    int rc = 0;
    auto mat = [&](void** p, size_t rows, size_t cols) { return dalloc(p, rows * cols * es); };
    auto vec = [&](float** p, size_t n) { return dalloc(p, n * sizeof(float)); };
    rc |= mat(&embed, V, W) | mat(&bigram, static_cast<size_t>(buckets) + 1, W) | mat(&head, V, W);
    rc |= vec(&fin_w, W) | vec(&fin_b, W) | vec(&fin_alpha, 1);
    for (size_t i = 0; i < spec.size() && !rc; ++i) {
      const LayerSpec& s = spec[i];
      LayerRun& r = run[i];
      if (s.mixer == MIX_LATENT) rc |= dalloc(&r.cache, static_cast<size_t>(e.num_blocks) * e.page * (s.kv_rank + s.rot_dim) * es);
      else rc |= dalloc(&r.state, static_cast<size_t>(e.num_slots) * s.heads * s.dim * s.vdim * sizeof(float));
      if (s.weights_of != static_cast<int>(i)) continue;
      LayerWeights& w = wts[i];
      rc |= mat(&w.w_in, s.n_in, W) | mat(&w.w_out, W, s.k_out);
      rc |= vec(&w.norm_w, W) | vec(&w.norm_b, W) | vec(&w.norm_alpha, 1);
      if (s.mixer == MIX_GLA) {
        rc |= mat(&w.a2, static_cast<size_t>(s.heads) * s.dim, s.a_rank) | vec(&w.a2_b, static_cast<size_t>(s.heads) * s.dim) | vec(&w.o_norm, s.vdim);
      } else {
        rc |= vec(&w.c_norm, s.kv_rank) | mat(&w.uk_t, static_cast<size_t>(s.heads) * s.kv_rank, s.dim) |
              mat(&w.uv, static_cast<size_t>(s.heads) * s.vdim, s.kv_rank);
        if (s.rot_dims > 0) {
          rc |= dalloc(&w.rope, static_cast<size_t>(e.max_model_len) * (s.rot_dims / 2) * sizeof(float2));
          if (!rc && rope_table_interleaved(w.rope, e.max_model_len, s.rot_dims, s.rot_base, e.stream)) rc = -2;
        }
      }
      if (s.ff_kind == FF_MOE)
        rc |= mat(&w.router, s.experts, W) | mat(&w.e_up, static_cast<size_t>(s.experts) * s.ff, W) | mat(&w.e_down, static_cast<size_t>(s.experts) * W, s.ff);
    }
    if (rc) return rc;
    const size_t T = e.Tcap;
    row_cap = static_cast<int>(std::min<size_t>(T, 256));
    rc |= dalloc(&x, T * W * sizeof(float)) | mat(&h, T, W) | mat(&inb, T, max_in) | mat(&ycat, T, max_kout) | mat(&ao, T, W) | mat(&fo, T, W) |
          mat(&hrow, row_cap, W);
    rc |= dalloc(&z, T * max_hd * sizeof(float)) | dalloc(&o32, T * max_hv * sizeof(float)) | dalloc(&qlat, T * max_ql * sizeof(float)) |
          dalloc(&olat, T * max_ol * sizeof(float)) | dalloc(&logits, static_cast<size_t>(row_cap) * V * sizeof(float));
    if (any_moe) {
      moe_cap = static_cast<int>((T * max_top + 63) / 64 * 64) + max_e * 64;
      rc |= dalloc(&scores, T * max_e * sizeof(float)) | dalloc(&topw, T * max_top * sizeof(float)) | dalloc(&topi, T * max_top * sizeof(int)) |
            dalloc(&sorted_rows, static_cast<size_t>(moe_cap) * sizeof(int)) | dalloc(&tile_group, static_cast<size_t>(moe_cap / 64) * sizeof(int)) |
            dalloc(&pair_pos, T * max_top * sizeof(int)) | mat(&eact, moe_cap, max_eff) | dalloc(&edown, static_cast<size_t>(moe_cap) * W * sizeof(float));
    }
    if (max_ol > 1 && dt == DT_BF16) {
      split_ws_floats = 1024ll * (max_ol + 2 * 64);   // rows x splits <= 1024 of [kv_rank + 2] per head
      rc |= dalloc(&split_ws, static_cast<size_t>(split_ws_floats) * sizeof(float));
    }
    if (rc) return rc;
    register_tensors();
    rc = setup_tc();
    if (rc) return rc;
    return cudaStreamSynchronize(e.stream) == cudaSuccess ? 0 : -2;
  }

  // The large projections of a bf16 model run on the tcgen05 pair GEMM (gemm2_tcgen05.cu) when their shapes allow it: the
  // input projection [n_in, width] and the output projection [width, k_out], K % 8 == 0.  B200_NX_TC=0 keeps every
  // projection on linear.cu (A/B knob); fp32 models always do.
  int setup_tc() {
    const char* ev = getenv("B200_NX_TC");
    use_tc = dt == DT_BF16 && !(ev && atoi(ev) == 0) && W % 8 == 0 && gemm_variant() == 2;
    if (!use_tc) return 0;
    int maxN = W, max_kout = 8;
    for (auto& s : spec) { maxN = std::max(maxN, s.n_in); max_kout = std::max(max_kout, s.k_out); }
    const size_t ws_bytes = std::max(gemm_workspace_bytes(env.sms), gemm_deferred_ws_bytes(env.sms));
    if (dalloc(&gemm_ws, ws_bytes)) return -3;
    const size_t n_counters = 2ull * (maxN / 128 + 2) * (env.Tcap / 32 + 2);
    if (dalloc(&gemm_counters, n_counters * sizeof(int))) return -3;
    const int bns[kGemmNumBlockN] = {32, 64, 128, 256, 512};
    for (int i = 0; i < kGemmNumBlockN; ++i)
      if (gemm_make_x_map(&xm_h[i], h, env.Tcap, W, W, bns[i])) { use_tc = false; return 0; }
    for (size_t i = 0; i < spec.size(); ++i) {
      const LayerSpec& s = spec[i];
      if (s.weights_of != static_cast<int>(i)) continue;
      LayerWeights& w = wts[i];
      w.tc_in = gemm_plan_init(&w.p_in, w.w_in, s.n_in, W, W, gemm_ws, gemm_counters, env.sms) == 0;
      if (w.tc_in) w.p_in.ws_bytes = ws_bytes;
      w.tc_out = s.k_out % 8 == 0 && gemm_plan_init(&w.p_out, w.w_out, W, s.k_out, s.k_out, gemm_ws, gemm_counters, env.sms) == 0;
      for (int j = 0; j < kGemmNumBlockN && w.tc_out; ++j)
        if (gemm_make_x_map(&w.xm_out[j], ycat, env.Tcap, s.k_out, s.k_out, bns[j])) w.tc_out = false;
      if (w.tc_out) w.p_out.ws_bytes = ws_bytes;
      if (s.ff_kind == FF_MOE && s.ff % 8 == 0) {
        w.p_eup.resize(s.experts);
        w.p_edown.resize(s.experts);
        bool ok = true;
        for (int e = 0; e < s.experts && ok; ++e) {
          ok = gemm_plan_init(&w.p_eup[e], static_cast<bf16*>(w.e_up) + static_cast<size_t>(e) * s.ff * W, s.ff, W, W, gemm_ws, gemm_counters, env.sms) == 0 &&
               gemm_plan_init(&w.p_edown[e], static_cast<bf16*>(w.e_down) + static_cast<size_t>(e) * W * s.ff, W, s.ff, s.ff, gemm_ws, gemm_counters, env.sms) == 0;
          w.p_eup[e].ws_bytes = w.p_edown[e].ws_bytes = ws_bytes;
        }
        if (!ok) { w.p_eup.clear(); w.p_edown.clear(); }
      }
    }
    if (moe_cap) {
      int max_e = 1;
      for (auto& s : spec) max_e = std::max(max_e, s.experts);
      if (dalloc(&hsorted, static_cast<size_t>(moe_cap) * W * 2) || dalloc(&edown16, static_cast<size_t>(moe_cap) * W * 2) ||
          dalloc(&expert_rows, static_cast<size_t>(max_e) * 2 * sizeof(int))) return -3;
      if (cudaMallocHost(&expert_rows_host, static_cast<size_t>(max_e) * 2 * sizeof(int)) != cudaSuccess) return -3;
    }
    return 0;
  }

  void reg(const std::string& name, void* p, size_t bytes) { tensors[name] = {p, bytes}; }
  void register_tensors() {
    const size_t es = dtype_bytes(dt);
    reg("embed", embed, static_cast<size_t>(V) * W * es);
    reg("bigram", bigram, (static_cast<size_t>(buckets) + 1) * W * es);
    reg("head", head, static_cast<size_t>(V) * W * es);
    for (size_t i = 0; i < spec.size(); ++i) {
      if (spec[i].weights_of != static_cast<int>(i)) continue;
      const std::string p = "l" + std::to_string(i) + ".";
      reg(p + "w_in", wts[i].w_in, static_cast<size_t>(spec[i].n_in) * W * es);
      reg(p + "w_out", wts[i].w_out, static_cast<size_t>(W) * spec[i].k_out * es);
    }
  }

  // ------------------------------------------------------------ weights
  // host fp32 [rows, cols] -> device rows [row0, row0 + rows) x columns [col0, col0 + cols) of a matrix with leading dimension ld
  int put(void* dst, size_t ld, size_t row0, size_t col0, const std::vector<float>& src, size_t rows, size_t cols) {
    const size_t es = dtype_bytes(dt);
    std::vector<uint8_t> tmp(rows * cols * es);
    if (dt == DT_F32) memcpy(tmp.data(), src.data(), tmp.size());
    else {
      bf16* o = reinterpret_cast<bf16*>(tmp.data());
      for (size_t i = 0; i < rows * cols; ++i) o[i] = __float2bfloat16_rn(src[i]);
    }
    uint8_t* d = static_cast<uint8_t*>(dst) + (row0 * ld + col0) * es;
    return cudaMemcpy2D(d, ld * es, tmp.data(), cols * es, cols * es, rows, cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -2;
  }
  int putf(float* dst, const std::vector<float>& src) {
    return cudaMemcpy(dst, src.data(), src.size() * sizeof(float), cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -2;
  }

  int load(const CheckpointReader& ck, std::string* err) override {
    std::vector<float> v;
    std::vector<int64_t> sh;
    auto get = [&](const std::string& name, int64_t rows, int64_t cols) {
      if (!ck.read_f32(name, &v, &sh, err)) return false;
      int64_t n = 1;
      for (auto d : sh) n *= d;
      const int64_t r = sh.size() == 2 ? sh[0] : 1, c = sh.size() == 2 ? sh[1] : n;
      if ((rows >= 0 && r != rows) || c != cols) {
        *err = name + ": shape [" + std::to_string(r) + "," + std::to_string(c) + "] does not fit the config";
        return false;
      }
      return true;
    };
    int rc = 0;
#define MAT(name, dst, ld, row0, col0, rows, cols) do { if (!get(name, rows, cols)) return -4; rc |= put(dst, ld, row0, col0, v, rows, cols); } while (0)
#define VEC(name, dst, n) do { if (!get(name, 1, n)) return -4; rc |= putf(dst, v); } while (0)
    MAT("embed", embed, W, 0, 0, V, W);
    MAT("bigram", bigram, W, 0, 0, buckets + 1, W);
    MAT("head", head, W, 0, 0, V, W);
    VEC("final.norm", fin_w, W); VEC("final.norm.b", fin_b, W); VEC("final.norm.alpha", fin_alpha, 1);
    for (size_t i = 0; i < spec.size(); ++i) {
      LayerSpec& s = spec[i];
      if (s.weights_of != static_cast<int>(i)) continue;
      LayerWeights& w = wts[i];
      const std::string p = "l" + std::to_string(i) + ".", m = p + "mix.", f = p + "mlp.";
      VEC(p + "norm1", w.norm_w, W); VEC(p + "norm1.b", w.norm_b, W); VEC(p + "norm1.alpha", w.norm_alpha, 1);
      const int HD = s.heads * s.dim, HV = s.heads * s.vdim;
      if (s.mixer == MIX_GLA) {
        if (!get(m + "a1", -1, W)) return -4;
        if (sh.size() != 2 || sh[0] != s.a_rank) { *err = m + "a1: " + std::to_string(sh.empty() ? 0 : sh[0]) + " rows, the engine was sized for " + std::to_string(s.a_rank); return -4; }
        rc |= put(w.w_in, W, s.off_a1, 0, v, s.a_rank, W);
        MAT(m + "q", w.w_in, W, s.off_q, 0, HD, W);
        MAT(m + "k", w.w_in, W, s.off_k, 0, HD, W);
        MAT(m + "v", w.w_in, W, s.off_v, 0, HV, W);
        MAT(m + "g", w.w_in, W, s.off_g, 0, HV, W);
        MAT(m + "a2", w.a2, s.a_rank, 0, 0, HD, s.a_rank);
        VEC(m + "a2.b", w.a2_b, HD);
        VEC(m + "norm", w.o_norm, s.vdim);
      } else {
        MAT(m + "q", w.w_in, W, s.off_q, 0, s.heads * (s.dim + s.rot_dim), W);
        MAT(m + "dkv", w.w_in, W, s.off_dkv, 0, s.kv_rank + s.rot_dim, W);
        MAT(m + "g", w.w_in, W, s.off_g, 0, HV, W);
        VEC(m + "dkv.norm", w.c_norm, s.kv_rank);
        if (!get(m + "uk", HD, s.kv_rank)) return -4;
        {
          // [heads * dim, kv_rank] -> per head [kv_rank, dim]
          std::vector<float> t(v.size());
          for (int hh = 0; hh < s.heads; ++hh)
            for (int d = 0; d < s.dim; ++d)
              for (int c = 0; c < s.kv_rank; ++c)
                t[(static_cast<size_t>(hh) * s.kv_rank + c) * s.dim + d] = v[(static_cast<size_t>(hh) * s.dim + d) * s.kv_rank + c];
          rc |= put(w.uk_t, s.dim, 0, 0, t, static_cast<size_t>(s.heads) * s.kv_rank, s.dim);
        }
        MAT(m + "uv", w.uv, s.kv_rank, 0, 0, HV, s.kv_rank);
      }
      MAT(m + "o", w.w_out, s.k_out, 0, 0, W, HV);
      if (s.ff_kind == FF_DENSE) {
        MAT(f + "gate", w.w_in, W, s.off_gu, 0, s.ff, W);
        MAT(f + "up", w.w_in, W, s.off_gu + s.ff, 0, s.ff, W);
        MAT(f + "down", w.w_out, s.k_out, 0, HV, W, s.ff);
      } else if (s.ff_kind == FF_MOE) {
        MAT(f + "router", w.router, W, 0, 0, s.experts, W);
        for (int e = 0; e < s.experts; ++e) {
          const std::string ep = f + "e" + std::to_string(e) + ".";
          MAT(ep + "up", w.e_up, W, static_cast<size_t>(e) * s.ff, 0, s.ff, W);
          MAT(ep + "down", w.e_down, s.ff, static_cast<size_t>(e) * W, 0, W, s.ff);
        }
      }
    }
#undef MAT
#undef VEC
    if (rc) { *err = "copying weights to the device failed"; return -2; }
    return 0;
  }

  // Seeded random weights of a plausible scale (benchmarks: there is no checkpoint of a real size).
  int randomize(uint64_t seed) override {
    cudaStream_t st = env.stream;
    int rc = 0;
    uint64_t k = seed * 1000003ull + 17;
    auto M = [&](void* p, size_t n, float sc) { rc |= fill_uniform(p, dt, n, ++k, sc, 0.f, st); };
    auto F = [&](float* p, size_t n, float sc, float off) { rc |= fill_uniform(p, DT_F32, n, ++k, sc, off, st); };
    const float sw = 1.7f / sqrtf(static_cast<float>(W));
    M(embed, static_cast<size_t>(V) * W, 1.0f); M(bigram, (static_cast<size_t>(buckets) + 1) * W, 0.5f); M(head, static_cast<size_t>(V) * W, sw);
    F(fin_w, W, 0.1f, 1.f); F(fin_b, W, 0.05f, 0.f); F(fin_alpha, 1, 0.f, 0.5f);
    for (size_t i = 0; i < spec.size(); ++i) {
      const LayerSpec& s = spec[i];
      if (s.weights_of != static_cast<int>(i)) continue;
      LayerWeights& w = wts[i];
      M(w.w_in, static_cast<size_t>(s.n_in) * W, sw);
      M(w.w_out, static_cast<size_t>(W) * s.k_out, 1.7f / sqrtf(static_cast<float>(s.k_out)));
      F(w.norm_w, W, 0.1f, 1.f); F(w.norm_b, W, 0.05f, 0.f); F(w.norm_alpha, 1, 0.f, 0.5f);
      if (s.mixer == MIX_GLA) {
        M(w.a2, static_cast<size_t>(s.heads) * s.dim * s.a_rank, 1.7f / sqrtf(static_cast<float>(s.a_rank)));
        F(w.a2_b, static_cast<size_t>(s.heads) * s.dim, 1.f, 3.f);
        F(w.o_norm, s.vdim, 0.1f, 1.f);
      } else {
        F(w.c_norm, s.kv_rank, 0.1f, 1.f);
        M(w.uk_t, static_cast<size_t>(s.heads) * s.kv_rank * s.dim, 1.7f / sqrtf(static_cast<float>(s.kv_rank)));
        M(w.uv, static_cast<size_t>(s.heads) * s.vdim * s.kv_rank, 1.7f / sqrtf(static_cast<float>(s.kv_rank)));
      }
      if (s.ff_kind == FF_MOE) {
        M(w.router, static_cast<size_t>(s.experts) * W, sw);
        M(w.e_up, static_cast<size_t>(s.experts) * s.ff * W, sw);
        M(w.e_down, static_cast<size_t>(s.experts) * W * s.ff, 1.7f / sqrtf(static_cast<float>(s.ff)));
      }
    }
    if (rc) return -2;
    return cudaStreamSynchronize(st) == cudaSuccess ? 0 : -2;
  }

  // ------------------------------------------------------------ forward
  int project(const GemmPlan& plan, bool tc, const CUtensorMap* xm, const void* X, const void* Wm, void* Y, int T, int N, int K) {
    static const int tc_min_t = [] { const char* e = getenv("B200_NX_TC_MIN_T"); return e ? atoi(e) : 1; }();   // A/B knob
    if (tc && T >= tc_min_t) {
      const int bn = gemm_block_n_for(T);
      return gemm_run(plan, xm[gemm_block_n_index(bn)], bn, Y, N, T, env.stream);
    }
    return linear(linear_args(X, dt, Wm, dt, Y, dt, T, N, K), env.stream);
  }

  // per-kernel device time (b200_engine_kernel_times): with profiling on, every launch is bracketed by events and waited for
  cudaEvent_t pe0 = nullptr, pe1 = nullptr;
  void prof_start() {
    if (!profile_kernels) return;
    if (!pe0) { cudaEventCreate(&pe0); cudaEventCreate(&pe1); }
    cudaEventRecord(pe0, env.stream);
  }
  void prof_stop(const char* name) {
    if (!profile_kernels) return;
    cudaEventRecord(pe1, env.stream);
    cudaEventSynchronize(pe1);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, pe0, pe1);
    auto& t = kernel_times[name];
    t.first += ms * 1000.0;
    t.second += 1;
  }
#define KRN(name, call) do { prof_start(); const int r_ = (call); if (r_ && !rc) { failed_kernel = name; failed_rc = r_; } rc |= r_; prof_stop(name); } while (0)
  const char* failed_kernel = "";
  int failed_rc = 0;

  int forward(const StepBatch& b, int* sampled, float* host_logits, int64_t* launches) override {
    cudaStream_t st = env.stream;
    const int T = b.T;
    int rc = 0;
    int64_t nl = 0;
    KRN("embed", embed_bigram(embed, bigram, dt, b.ids, b.prev_ids, x, T, W, V, buckets, mul_prev, mul_cur, st));
    const LayerWeights& w0 = wts[spec[0].weights_of];
    KRN("residual_norm", residual_dyt(x, nullptr, nullptr, dt, 0.f, w0.norm_w, w0.norm_b, w0.norm_alpha, h, dt, nullptr, T, W, st));
    nl += 2;
    for (size_t li = 0; li < spec.size() && !rc; ++li) {
      const LayerSpec& s = spec[li];
      const LayerWeights& w = wts[s.weights_of];
      const LayerRun& r = run[li];
      const int HV = s.heads * s.vdim;
      KRN("proj_in", project(w.p_in, w.tc_in, xm_h, h, w.w_in, inb, T, s.n_in, W));
      ++nl;
      const size_t es = dtype_bytes(dt);
      auto col = [&](void* base, size_t off) { return static_cast<void*>(static_cast<uint8_t*>(base) + off * es); };
      if (s.mixer == MIX_GLA) {
        LinearArgs la = linear_args(col(inb, s.off_a1), dt, w.a2, dt, z, DT_F32, T, s.heads * s.dim, s.a_rank);
        la.ldx = s.n_in;
        KRN("gla_decay_proj", linear(la, st));
        GlaArgs g;
        g.qkv = inb; g.t = dt; g.ld = s.n_in; g.q_off = s.off_q; g.k_off = s.off_k; g.v_off = s.off_v;
        g.z = z; g.T = T; g.z_bias = w.a2_b; g.inv_tau = 1.0f / s.tau; g.q_scale = 1.0f / sqrtf(static_cast<float>(s.dim));
        g.states = r.state; g.seqs = b.seqs; g.nseq = b.nseq;
        g.heads = s.heads; g.dim = s.dim; g.vdim = s.vdim; g.o = o32;
        KRN("gla_scan", gla_scan(g, st));
        KRN("gla_out_gate", gla_out_gate(o32, col(inb, s.off_g), s.n_in, w.o_norm, eps, ycat, s.k_out, dt, T, s.heads, s.vdim, st));
        nl += 3;
      } else {
        const int C = s.kv_rank, R = s.rot_dim, E = C + R;
        LatentPrepArgs p;
        p.q = col(inb, s.off_q); p.ldq = s.n_in; p.dkv = col(inb, s.off_dkv); p.lddkv = s.n_in; p.t = dt;
        p.norm_w = w.c_norm; p.eps = eps; p.rope = w.rope; p.rot_dims = s.rot_dims;
        p.positions = b.pos; p.slots = b.slots; p.cache = r.cache; p.qlat = qlat;
        p.T = T; p.heads = s.heads; p.dim = s.dim; p.rot_dim = R; p.kv_rank = C;
        KRN("latent_prep", latent_prep(p, st));
        // latent query: per head [T, dim] x [kv_rank, dim]^T into the head's first kv_rank columns of qlat
        LinearArgs lq = linear_args(col(inb, s.off_q), dt, w.uk_t, dt, qlat, DT_F32, T, C, s.dim);
        lq.ldx = s.n_in; lq.ldy = s.heads * E; lq.batch = s.heads; lq.xbs = s.dim + R; lq.wbs = static_cast<long long>(C) * s.dim; lq.ybs = E;
        KRN("latent_q_absorb", linear(lq, st));
        LatentAttnArgs a;
        a.qlat = qlat; a.cache = r.cache; a.t = dt; a.positions = b.pos; a.seq_of_tok = b.seq_of_tok; a.block_tables = b.btab;
        a.max_blocks = b.max_blocks; a.page = env.page; a.olat = olat;
        a.T = T; a.heads = s.heads; a.kv_rank = C; a.rot_dim = R; a.window = std::min(s.window, env.max_model_len); a.scale = s.scale;
        a.seqs = b.seqs; a.nseq = b.nseq; a.max_ctx = b.max_ctx; a.split_ws = split_ws; a.split_ws_floats = split_ws_floats;
        KRN("latent_attention", latent_attention(a, st));
        // values: per head [T, kv_rank] x [vdim, kv_rank]^T into the head's columns of the output projection's input
        LinearArgs lv = linear_args(olat, DT_F32, w.uv, dt, ycat, dt, T, s.vdim, C);
        lv.ldx = s.heads * C; lv.ldy = s.k_out; lv.batch = s.heads; lv.xbs = C; lv.wbs = static_cast<long long>(s.vdim) * C; lv.ybs = s.vdim;
        KRN("latent_v_expand", linear(lv, st));
        KRN("sigmoid_gate", sigmoid_gate(ycat, s.k_out, col(inb, s.off_g), s.n_in, dt, T, HV, st));
        nl += 5;
      }
      if (s.ff_kind == FF_DENSE) {
        KRN("glu", glu_clamped(col(inb, s.off_gu), s.n_in, col(ycat, HV), s.k_out, dt, T, s.ff, s.limit, 1.702f, st));
        ++nl;
      }
      KRN("proj_out", project(w.p_out, w.tc_out, w.xm_out, ycat, w.w_out, ao, T, W, s.k_out));
      ++nl;
      const void* f_out = nullptr;
      if (s.ff_kind == FF_MOE) {
        KRN("moe_router", linear(linear_args(h, dt, w.router, dt, scores, DT_F32, T, s.experts, W), st));
        KRN("moe_route", moe_route(scores, topi, topw, T, s.experts, s.groups, s.keep, s.top, st));
        const int cap = (T * s.top + 63) / 64 * 64 + s.experts * 64;
        const char* mte = getenv("B200_NX_MOE_TC_MIN_T");   // A/B knob
        const int moe_tc_min = mte ? atoi(mte) : 256;
        const bool per_expert = !w.p_eup.empty() && T >= moe_tc_min;
        KRN("moe_align", moe_align(topi, T, s.top, s.experts, sorted_rows, tile_group, pair_pos, cap, st, per_expert ? expert_rows : nullptr));
        if (per_expert) {
          // Large steps: every expert's rows are one tcgen05 GEMM.  The row counts come back to the host (one small copy
          // and a wait per layer, paid only by steps of hundreds of tokens), the inputs are gathered into sorted order.
          KRN("moe_gather", moe_gather_bf16(h, sorted_rows, hsorted, cap, W, st));
          if (cudaMemcpyAsync(expert_rows_host, expert_rows, static_cast<size_t>(s.experts) * 2 * sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
              cudaStreamSynchronize(st) != cudaSuccess) rc = -2;
          prof_start();
          for (int e = 0; e < s.experts && !rc; ++e) {
            const int start = expert_rows_host[2 * e], cnt = expert_rows_host[2 * e + 1];
            if (cnt <= 0) continue;
            const int bn = gemm_block_n_for(cnt);
            CUtensorMap tm;
            if (gemm_make_x_map(&tm, static_cast<bf16*>(hsorted) + static_cast<size_t>(start) * W, cnt, W, W, bn)) { rc = -2; break; }
            rc |= gemm_run(w.p_eup[e], tm, bn, static_cast<bf16*>(eact) + static_cast<size_t>(start) * s.ff, s.ff, cnt, st);
            ++nl;
          }
          prof_stop("moe_up");
          KRN("moe_act", relu2_bf16(eact, static_cast<long long>(cap) * s.ff, st));
          prof_start();
          for (int e = 0; e < s.experts && !rc; ++e) {
            const int start = expert_rows_host[2 * e], cnt = expert_rows_host[2 * e + 1];
            if (cnt <= 0) continue;
            const int bn = gemm_block_n_for(cnt);
            CUtensorMap tm;
            if (gemm_make_x_map(&tm, static_cast<bf16*>(eact) + static_cast<size_t>(start) * s.ff, cnt, s.ff, s.ff, bn)) { rc = -2; break; }
            rc |= gemm_run(w.p_edown[e], tm, bn, static_cast<bf16*>(edown16) + static_cast<size_t>(start) * W, W, cnt, st);
            ++nl;
          }
          prof_stop("moe_down");
          KRN("moe_combine", moe_combine(edown16, DT_BF16, pair_pos, topw, fo, dt, T, s.top, W, st));
          nl += 5;
        } else if (T * s.top <= 64) {
          // decode-sized steps: one weight-streaming pass per chosen (token, expert) pair
          LinearArgs up = linear_args(h, dt, w.e_up, dt, eact, dt, T * s.top, s.ff, W);
          up.wbs = static_cast<long long>(s.ff) * W; up.act = LIN_RELU2;
          const PickedRows pu = {T * s.top, nullptr, s.top, pair_pos, topi};
          KRN("moe_up", linear_picked_rows(up, pu, st));
          LinearArgs dn = linear_args(eact, dt, w.e_down, dt, edown, DT_F32, T * s.top, W, s.ff);
          dn.wbs = static_cast<long long>(W) * s.ff;
          const PickedRows pd = {T * s.top, pair_pos, 1, pair_pos, topi};
          KRN("moe_down", linear_picked_rows(dn, pd, st));
          KRN("moe_combine", moe_combine(edown, DT_F32, pair_pos, topw, fo, dt, T, s.top, W, st));
          nl += 4;
        } else {
          LinearArgs up = linear_args(h, dt, w.e_up, dt, eact, dt, cap, s.ff, W);
          up.x_rows = sorted_rows; up.tile_group = tile_group; up.wbs = static_cast<long long>(s.ff) * W; up.act = LIN_RELU2;
          KRN("moe_up", linear(up, st));
          LinearArgs dn = linear_args(eact, dt, w.e_down, dt, edown, DT_F32, cap, W, s.ff);
          dn.tile_group = tile_group; dn.wbs = static_cast<long long>(W) * s.ff;
          KRN("moe_down", linear(dn, st));
          KRN("moe_combine", moe_combine(edown, DT_F32, pair_pos, topw, fo, dt, T, s.top, W, st));
          nl += 4;
        }
        f_out = fo;
        nl += 2;
      }
      const bool last = li + 1 == spec.size();
      const LayerWeights* nw = last ? nullptr : &wts[spec[li + 1].weights_of];
      KRN("residual_norm", residual_dyt(x, ao, f_out, dt, mult, nw ? nw->norm_w : nullptr, nw ? nw->norm_b : nullptr, nw ? nw->norm_alpha : nullptr,
                         last ? nullptr : h, dt, nullptr, T, W, st));
      ++nl;
      if (residual_sink && !rc) {
        const size_t at = residual_sink->size();
        residual_sink->resize(at + static_cast<size_t>(T) * W);
        if (cudaMemcpyAsync(residual_sink->data() + at, x, static_cast<size_t>(T) * W * sizeof(float), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess) rc = -2;
      }
    }
    // head: final norm of the wanted rows, logits in fp32, greedy choice; in chunks of row_cap rows
    for (int r0 = 0; r0 < b.S && !rc; r0 += row_cap) {
      const int n = std::min(row_cap, b.S - r0);
      KRN("residual_norm", residual_dyt(x, nullptr, nullptr, dt, 0.f, fin_w, fin_b, fin_alpha, hrow, dt, b.rows + r0, n, W, st));
      KRN("head", linear(linear_args(hrow, dt, head, dt, logits, DT_F32, n, V, W), st));
      KRN("argmax", argmax_f32(logits, sampled + r0, n, V, st));
      nl += 3;
      if (host_logits && cudaMemcpyAsync(host_logits + static_cast<size_t>(r0) * V, logits, static_cast<size_t>(n) * V * sizeof(float),
                                         cudaMemcpyDeviceToHost, st) != cudaSuccess) rc = -2;
    }
    if (launches) *launches += nl;
    if (rc) { set_error("Nomanex forward: %s failed with %d (%s)", failed_kernel, failed_rc, cudaGetErrorString(cudaGetLastError())); return -2; }
    return 0;
  }
};

}  // namespace

#undef KRN

std::unique_ptr<Model> make_nomanex(const JVal& config, DType dtype, std::string* err) {
  std::unique_ptr<Nomanex> m(new Nomanex(dtype));
  if (!m->parse(config, err)) return nullptr;
  return std::unique_ptr<Model>(m.release());
}

}  // namespace b200
