// Zinavik: a decoder-only design on several fp32 residual streams (hyper-connections) whose mixer is two branches side by
// side on the same normed input, and whose feed-forward is a mixture of clamped gated experts with a shared expert.
//
//   x_s[t]   = embed[token] * scale                                 for every stream s
//   sublayer : u = sum_s in[s] x_s;  y = f(rmsnorm(u));  x_j <- sum_s mix[s, j] x_s + out[j] y        (hyper.cu)
//   mixer    = a_l * left(h) + a_r * right(h)
//     left   : softmax attention, grouped key/value heads, rotary positions (interleaved pairs, YaRN scaling) on the
//              first rot.dims dimensions, q and k of every head divided by their RMS, sliding window that also keeps the
//              first tokens, sigmoid output gate                                             (window_attention.cu)
//     right  : linear attention with one constant decay per head on silu(q), silu(k), silu(v), RMS norm over the
//              concatenated heads, sigmoid output gate                                        (gla.cu, head_decay form)
//   ff       = sum over the `top` experts with the largest sigmoid router scores of expert(score * h)
//              + sigmoid(w_sg . h) * shared(h),   expert(h) = W_down (g * sigmoid(1.702 g) * (u + 1)),
//              g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit)                      (moe.cu, linear.cu)
//   logits   = embed rmsnorm(sum_s x_s)                              (the embedding table, without its scale)
// A range of layers may run several times in a row with the same weights (`loop`); every run has its own key/value
// cache and recurrent state.
//
// Per layer run the kernel sequence is: ONE input projection for everything that reads the mixer's normed input (left
// q, k, v, gate and right q, k, v, gate concatenated row-wise at load), rotation + norm + cache write, the two mixers
// (each writes its gated, branch-scaled heads into its column block of one buffer), ONE output projection over
// [left heads | right heads] (W_o of both branches concatenated column-wise, so the weighted sum of the branches comes
// out of the accumulator), then the stream update fused with the next sublayer's read and norm.  Every size and
// constant comes from config.json; matrices and activations are bf16 or fp32, with the streams, norms, softmax,
// router, decays and recurrent state in fp32 either way.
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

struct LeftSpec {
  int heads = 0, kv_heads = 0, dim = 0, vdim = 0;
  int window = 1 << 30, keep_first = 0;
  int rot_dims = 0;
  double rot_base = 10000.0;
  bool yarn = false;
  RopeYarn ys = {1.0, 1.0, 1.0, 1.0};
  float scale = 1.f;
};
struct RightSpec {
  int heads = 0, dim = 0, vdim = 0;
  std::vector<float> decay;
};
struct LayerSpec {
  LeftSpec l;
  RightSpec r;
  float left_scale = 1.f, right_scale = 1.f;
  bool mlp = false, shared = false;
  int experts = 0, top = 0, ff = 0, sff = 0;
  float limit = 0.f, slimit = 0.f;
  // column layout of the input projection's output row, of the output projection's input row and of the shared expert's row
  int n_in = 0, off_lq = 0, off_lk = 0, off_lv = 0, off_lg = 0, off_rq = 0, off_rk = 0, off_rv = 0, off_rg = 0;
  int k_out = 0, hv_l = 0, hv_r = 0;
  int n_sh = 0;
};

struct Hyper {   // one sublayer's stream weights (device, fp32); null when the model has a single plain residual
  float *in = nullptr, *out = nullptr, *mix = nullptr;
};

struct LayerWeights {
  void* w_in = nullptr;    // [n_in, width]
  void* w_out = nullptr;   // [width, k_out]
  float *norm1 = nullptr, *norm2 = nullptr, *r_norm = nullptr, *decay = nullptr;
  float2* rope = nullptr;  // [max_model_len][rot_dims / 2]
  Hyper hc1, hc2;
  void* router = nullptr;  // [experts (+ 1), width]: the router rows, then the shared expert's gate row (its logit comes out in fp32 too)
  void* e_gu = nullptr;    // [experts][2 ff][width]  gate rows, then up rows
  void* e_down = nullptr;  // [experts][width][ff]
  void* sh_in = nullptr;   // [n_sh, width]: gate [sff] | up [sff]
  void* sh_down = nullptr; // [width, sff]
  GemmPlan p_in, p_out, p_shin, p_shdown;
  std::vector<GemmPlan> p_egu, p_edown;
  CUtensorMap xm_out[kGemmNumBlockN], xm_shact[kGemmNumBlockN];
  bool tc_in = false, tc_out = false, tc_shin = false, tc_shdown = false;
};

struct LayerRun {
  int layer = 0;
  void* cache = nullptr;    // [num_blocks * page][kv_heads * (dim + vdim)]
  float* state = nullptr;   // [slots][heads][dim][vdim]
};

bool jnum(const JVal* o, const char* k, double* out) {
  const JVal* v = o ? o->get(k) : nullptr;
  if (!v || v->type != JVal::Num) return false;
  *out = v->num;
  return true;
}

class Zinavik : public Model {
 public:
  DType dt;
  int V = 0, W = 0, ns = 1;
  bool hyper = false;     // the config names `streams`: every sublayer has stream weights
  float eps = 1e-5f, emb_scale = 1.f;
  std::vector<LayerSpec> spec;
  std::vector<LayerWeights> wts;
  std::vector<LayerRun> run;     // the order the layers run in, loops unrolled
  ModelEnv env;
  void* embed = nullptr;
  float* fin_w = nullptr;
  // activations
  float* x = nullptr;            // [ns][Tcap][W]
  long long xstride = 0;
  void *h = nullptr, *inb = nullptr, *ycat = nullptr, *ao = nullptr, *fo = nullptr, *hrow = nullptr;
  void *egu = nullptr, *eact = nullptr, *sh = nullptr, *shact = nullptr, *sdown = nullptr;
  float *qn = nullptr, *o32 = nullptr, *scores = nullptr, *topw = nullptr, *sorted_w = nullptr, *edown = nullptr, *logits = nullptr,
        *sumbuf = nullptr;
  int *topi = nullptr, *sorted_rows = nullptr, *tile_group = nullptr, *pair_pos = nullptr, *iota = nullptr;
  int row_cap = 0, moe_cap = 0;
  void *hsorted = nullptr, *edown16 = nullptr;
  int *expert_rows = nullptr, *expert_rows_host = nullptr;
  std::vector<void*> allocs;
  float* gemm_ws = nullptr;
  int* gemm_counters = nullptr;
  CUtensorMap xm_h[kGemmNumBlockN];
  bool use_tc = false;

  explicit Zinavik(DType d) : dt(d) {}
  ~Zinavik() override {
    for (auto& w : wts) {
      if (w.tc_in) gemm_plan_destroy(&w.p_in);
      if (w.tc_out) gemm_plan_destroy(&w.p_out);
      if (w.tc_shin) gemm_plan_destroy(&w.p_shin);
      if (w.tc_shdown) gemm_plan_destroy(&w.p_shdown);
      for (auto& p : w.p_egu) gemm_plan_destroy(&p);
      for (auto& p : w.p_edown) gemm_plan_destroy(&p);
    }
    if (expert_rows_host) cudaFreeHost(expert_rows_host);
    for (void* p : allocs) cudaFree(p);
  }
  const char* arch() const override { return "Zinavik"; }
  int vocab() const override { return V; }

  size_t cache_bytes_per_block(int page) const override {
    size_t b = 0;
    for (auto& r : run) {
      const LeftSpec& l = spec[r.layer].l;
      b += static_cast<size_t>(page) * l.kv_heads * (l.dim + l.vdim) * dtype_bytes(dt);
    }
    return b;
  }
  size_t state_bytes_per_slot() const override {
    size_t b = 0;
    for (auto& r : run) {
      const RightSpec& s = spec[r.layer].r;
      b += static_cast<size_t>(s.heads) * s.dim * s.vdim * sizeof(float);
    }
    return b;
  }
  int cache_window() const override {
    int w = 0;
    for (auto& s : spec) {
      if (s.l.window >= (1 << 30)) return 0;
      w = std::max(w, s.l.window);
    }
    return w;
  }
  int cache_keep_first() const override {
    int k = 0;
    for (auto& s : spec) k = std::max(k, s.l.keep_first);
    return k;
  }

  // ------------------------------------------------------------ config.json
  bool parse(const JVal& c, std::string* err) {
    double d = 0;
    auto whole = [&](const JVal* o, const char* k, int lo, int* out, const std::string& where) {
      double v = 0;
      if (!jnum(o, k, &v) || v < lo || v != floor(v) || v > 2147483647.0) { *err = "config: " + where + k; return false; }
      *out = static_cast<int>(v);
      return true;
    };
    if (!whole(&c, "vocab", 1, &V, "") || !whole(&c, "width", 1, &W, "")) return false;
    if (jnum(c.get("norm"), "eps", &d)) eps = static_cast<float>(d);
    if (jnum(c.get("embedding"), "scale", &d)) emb_scale = static_cast<float>(d);
    if (const JVal* sv = c.get("streams")) {
      if (!sv->is_null()) {
        if (!whole(&c, "streams", 1, &ns, "") || ns > 8) { *err = "config: streams (1..8)"; return false; }
        hyper = true;
      }
    }
    const JVal* ls = c.get("layers");
    if (!ls || ls->type != JVal::Arr || ls->arr.empty()) { *err = "config: layers"; return false; }
    for (size_t i = 0; i < ls->arr.size(); ++i) {
      const JVal& L = ls->arr[i];
      const std::string where = "layer " + std::to_string(i) + " ";
      LayerSpec s;
      const JVal* ty = L.get("type");
      if (!ty || ty->type != JVal::Str) { *err = "config: " + where + "type"; return false; }
      if (ty->str != "parallel") { *err = "config: unknown mixer \"" + ty->str + "\""; return false; }
      const JVal* mx = L.get("mixer");
      const JVal* lf = mx ? mx->get("left") : nullptr;
      const JVal* rt = mx ? mx->get("right") : nullptr;
      if (!lf || lf->type != JVal::Obj || !rt || rt->type != JVal::Obj) { *err = "config: " + where + "mixer.left / mixer.right"; return false; }
      if (jnum(mx, "left_scale", &d)) s.left_scale = static_cast<float>(d);
      if (jnum(mx, "right_scale", &d)) s.right_scale = static_cast<float>(d);
      LeftSpec& l = s.l;
      if (!whole(lf, "heads", 1, &l.heads, where + "left.") || !whole(lf, "dim", 1, &l.dim, where + "left.") || !whole(lf, "vdim", 1, &l.vdim, where + "left.")) return false;
      l.kv_heads = l.heads;
      if (lf->get("kv_heads") && !whole(lf, "kv_heads", 1, &l.kv_heads, where + "left.")) return false;
      if (l.heads % l.kv_heads) { *err = "config: " + where + "left.heads is no multiple of kv_heads"; return false; }
      if (l.vdim > 256) { *err = "config: " + where + "left.vdim above 256"; return false; }
      l.scale = 1.0f / sqrtf(static_cast<float>(l.dim));
      if (jnum(lf, "scale", &d)) l.scale = static_cast<float>(d);
      if (const JVal* mk = lf->get("mask")) {
        if (jnum(mk, "size", &d) && d >= 1) l.window = static_cast<int>(std::min(d, 1073741824.0));
        if (jnum(mk, "keep_first", &d) && d >= 0) l.keep_first = static_cast<int>(std::min(d, 1073741824.0));
      }
      if (const JVal* rot = lf->get("rot")) {
        if (rot->type == JVal::Obj) {
          l.rot_dims = l.dim / 2 * 2;
          if (rot->get("dims") && !whole(rot, "dims", 0, &l.rot_dims, where + "left.rot.")) return false;
          if (jnum(rot, "base", &d)) l.rot_base = d;
          if (l.rot_dims > l.dim || l.rot_dims % 2 || !(l.rot_base > 0)) { *err = "config: " + where + "left.rot"; return false; }
          const JVal* sc = rot->get("scaling");
          if (sc && sc->type == JVal::Obj) {
            l.yarn = true;
            if (!jnum(sc, "factor", &l.ys.factor) || !jnum(sc, "original", &l.ys.original) || !jnum(sc, "fast", &l.ys.fast) ||
                !jnum(sc, "slow", &l.ys.slow) || !(l.ys.factor > 0 && l.ys.original > 0 && l.ys.fast > 0 && l.ys.slow > 0)) {
              *err = "config: " + where + "left.rot.scaling"; return false;
            }
          }
        }
      }
      RightSpec& r = s.r;
      if (!whole(rt, "heads", 1, &r.heads, where + "right.") || !whole(rt, "dim", 1, &r.dim, where + "right.") || !whole(rt, "vdim", 1, &r.vdim, where + "right.")) return false;
      if (r.dim > 1024) { *err = "config: " + where + "right.dim above 1024"; return false; }
      const JVal* dc = rt->get("decay");
      if (dc && dc->type == JVal::Num) r.decay.assign(r.heads, static_cast<float>(dc->num));
      else if (dc && dc->type == JVal::Arr && static_cast<int>(dc->arr.size()) == r.heads) {
        for (auto& v : dc->arr) {
          if (v.type != JVal::Num) { *err = "config: " + where + "right.decay"; return false; }
          r.decay.push_back(static_cast<float>(v.num));
        }
      } else { *err = "config: " + where + "right.decay (one number per head)"; return false; }
      const JVal* mlp = L.get("mlp");
      if (mlp && mlp->type == JVal::Obj) {
        const JVal* kind = mlp->get("kind");
        if (!kind || kind->type != JVal::Str || kind->str != "moe") { *err = "config: " + where + "mlp.kind (moe)"; return false; }
        s.mlp = true;
        const JVal* ex = mlp->get("expert");
        const JVal* ro = mlp->get("router");
        if (!whole(ex, "ff", 1, &s.ff, where + "mlp.expert.") || !whole(ro, "experts", 1, &s.experts, where + "mlp.router.") ||
            !whole(ro, "top", 1, &s.top, where + "mlp.router.")) return false;
        if (s.top > s.experts) { *err = "config: " + where + "mlp.router.top above experts"; return false; }
        if (!jnum(ex, "limit", &d)) { *err = "config: " + where + "mlp.expert.limit"; return false; }
        s.limit = static_cast<float>(d);
        const JVal* sh = mlp->get("shared");
        if (sh && sh->type == JVal::Obj) {
          s.shared = true;
          if (!whole(sh, "ff", 1, &s.sff, where + "mlp.shared.")) return false;
          if (!jnum(sh, "limit", &d)) { *err = "config: " + where + "mlp.shared.limit"; return false; }
          s.slimit = static_cast<float>(d);
        }
      }
      layout(s);
      spec.push_back(s);
    }
    // the order of the runs: layers before the loop, the looped range `times` times, the rest
    const int n = static_cast<int>(spec.size());
    int start = 0, stop = 0, times = 1;
    if (const JVal* lp = c.get("loop")) {
      if (lp->type == JVal::Obj) {
        if (!whole(lp, "start", 0, &start, "loop.") || !whole(lp, "stop", 0, &stop, "loop.") || !whole(lp, "times", 1, &times, "loop.")) return false;
        if (start > stop || stop > n) { *err = "config: loop range outside the layers"; return false; }
      }
    }
    auto add = [&](int li) { LayerRun r; r.layer = li; run.push_back(r); };
    for (int i = 0; i < start; ++i) add(i);
    for (int k = 0; k < times; ++k)
      for (int i = start; i < stop; ++i) add(i);
    for (int i = stop; i < n; ++i) add(i);
    return true;
  }

  static int up8(int v) { return (v + 7) / 8 * 8; }
  void layout(LayerSpec& s) {
    int at = 0;
    auto block = [&](int* off, int n) { *off = at; at = up8(at + n); };   // every block starts 16-byte aligned
    block(&s.off_lq, s.l.heads * s.l.dim);
    block(&s.off_lk, s.l.kv_heads * s.l.dim);
    block(&s.off_lv, s.l.kv_heads * s.l.vdim);
    block(&s.off_lg, s.l.heads * s.l.vdim);
    block(&s.off_rq, s.r.heads * s.r.dim);
    block(&s.off_rk, s.r.heads * s.r.dim);
    block(&s.off_rv, s.r.heads * s.r.vdim);
    block(&s.off_rg, s.r.heads * s.r.vdim);
    s.n_in = at;
    s.hv_l = s.l.heads * s.l.vdim;
    s.hv_r = s.r.heads * s.r.vdim;
    s.k_out = s.hv_l + s.hv_r;
    s.n_sh = s.shared ? up8(2 * s.sff) : 0;
  }

  template <typename P>
  int dalloc(P** p, size_t bytes) {
    void* q = nullptr;
    if (cudaMalloc(&q, std::max<size_t>(bytes, 16)) != cudaSuccess) { set_error("Zinavik: device allocation of %zu bytes failed", bytes); return -3; }
    cudaMemsetAsync(q, 0, std::max<size_t>(bytes, 16), env.stream);
    allocs.push_back(q);
    *p = static_cast<P*>(q);
    return 0;
  }

  int init(const ModelEnv& e) override {
    env = e;
    const size_t es = dtype_bytes(dt);
    wts.resize(spec.size());
    int max_in = 8, max_kout = 8, max_qn = 1, max_hvr = 1, max_e = 1, max_top = 1, max_ff = 1, max_nsh = 8, max_sff = 1;
    bool any_moe = false, any_shared = false;
    for (auto& s : spec) {
      max_in = std::max(max_in, s.n_in);
      max_kout = std::max(max_kout, s.k_out);
      max_qn = std::max(max_qn, s.l.heads * s.l.dim);
      max_hvr = std::max(max_hvr, s.hv_r);
      if (s.mlp) {
        any_moe = true;
        max_e = std::max(max_e, s.experts + 1); max_top = std::max(max_top, s.top); max_ff = std::max(max_ff, s.ff);
        if (s.shared) { any_shared = true; max_nsh = std::max(max_nsh, s.n_sh); max_sff = std::max(max_sff, s.sff); }
      }
    }
    int rc = 0;
    auto mat = [&](void** p, size_t rows, size_t cols) { return dalloc(p, rows * cols * es); };
    auto vec = [&](float** p, size_t n) { return dalloc(p, n * sizeof(float)); };
    rc |= mat(&embed, V, W) | vec(&fin_w, W);
    for (auto& r : run) {
      const LayerSpec& s = spec[r.layer];
      rc |= dalloc(&r.cache, static_cast<size_t>(e.num_blocks) * e.page * s.l.kv_heads * (s.l.dim + s.l.vdim) * es);
      rc |= dalloc(&r.state, static_cast<size_t>(e.num_slots) * s.r.heads * s.r.dim * s.r.vdim * sizeof(float));
      if (rc) return rc;
    }
    for (size_t i = 0; i < spec.size() && !rc; ++i) {
      const LayerSpec& s = spec[i];
      LayerWeights& w = wts[i];
      rc |= mat(&w.w_in, s.n_in, W) | mat(&w.w_out, W, s.k_out) | vec(&w.norm1, W) | vec(&w.r_norm, s.hv_r) | vec(&w.decay, s.r.heads);
      if (!rc && cudaMemcpyAsync(w.decay, s.r.decay.data(), s.r.heads * sizeof(float), cudaMemcpyHostToDevice, e.stream) != cudaSuccess) rc = -2;
      if (s.l.rot_dims > 0) {
        rc |= dalloc(&w.rope, static_cast<size_t>(e.max_model_len) * (s.l.rot_dims / 2) * sizeof(float2));
        if (!rc && rope_table_yarn(w.rope, e.max_model_len, s.l.rot_dims, s.l.rot_base, s.l.yarn ? &s.l.ys : nullptr, e.stream)) rc = -2;
      }
      if (hyper) rc |= vec(&w.hc1.in, ns) | vec(&w.hc1.out, ns) | vec(&w.hc1.mix, static_cast<size_t>(ns) * ns);
      if (s.mlp) {
        rc |= vec(&w.norm2, W) | mat(&w.router, s.experts + (s.shared ? 1 : 0), W) | mat(&w.e_gu, static_cast<size_t>(s.experts) * 2 * s.ff, W) |
              mat(&w.e_down, static_cast<size_t>(s.experts) * W, s.ff);
        if (hyper) rc |= vec(&w.hc2.in, ns) | vec(&w.hc2.out, ns) | vec(&w.hc2.mix, static_cast<size_t>(ns) * ns);
        if (s.shared) rc |= mat(&w.sh_in, s.n_sh, W) | mat(&w.sh_down, W, s.sff);
      }
    }
    if (rc) return rc;
    const size_t T = e.Tcap;
    row_cap = static_cast<int>(std::min<size_t>(T, 256));
    xstride = static_cast<long long>(T) * W;
    rc |= dalloc(&x, static_cast<size_t>(ns) * T * W * sizeof(float)) | mat(&h, T, W) | mat(&inb, T, max_in) | mat(&ycat, T, max_kout) | mat(&ao, T, W) |
          mat(&hrow, row_cap, W);
    rc |= dalloc(&qn, T * max_qn * sizeof(float)) | dalloc(&o32, T * max_hvr * sizeof(float)) | dalloc(&logits, static_cast<size_t>(row_cap) * V * sizeof(float));
    if (any_moe) {
      moe_cap = static_cast<int>((T * max_top + 63) / 64 * 64) + max_e * 64;
      rc |= mat(&fo, T, W) | dalloc(&scores, T * max_e * sizeof(float)) | dalloc(&topw, T * max_top * sizeof(float)) | dalloc(&topi, T * max_top * sizeof(int)) |
            dalloc(&sorted_rows, static_cast<size_t>(moe_cap) * sizeof(int)) | dalloc(&tile_group, static_cast<size_t>(moe_cap / 64) * sizeof(int)) |
            dalloc(&pair_pos, T * max_top * sizeof(int)) | dalloc(&sorted_w, static_cast<size_t>(moe_cap) * sizeof(float)) |
            mat(&egu, moe_cap, 2 * static_cast<size_t>(max_ff)) | mat(&eact, moe_cap, max_ff) | dalloc(&edown, static_cast<size_t>(moe_cap) * W * sizeof(float)) |
            dalloc(&iota, static_cast<size_t>(64) * sizeof(int));
      if (!rc) {
        int hi[64];
        for (int i = 0; i < 64; ++i) hi[i] = i;
        if (cudaMemcpyAsync(iota, hi, sizeof(hi), cudaMemcpyHostToDevice, e.stream) != cudaSuccess || cudaStreamSynchronize(e.stream) != cudaSuccess) rc = -2;
      }
      if (any_shared) rc |= mat(&sh, T, max_nsh) | mat(&shact, T, max_sff) | mat(&sdown, T, W);
    }
    if (rc) return rc;
    register_tensors();
    rc = setup_tc();
    if (rc) return rc;
    return cudaStreamSynchronize(e.stream) == cudaSuccess ? 0 : -2;
  }

  // The projections of a bf16 model run on the tcgen05 pair GEMM (gemm2_tcgen05.cu) where their shapes allow it (K % 8 == 0):
  // input and output projection, the shared expert, and every expert for steps large enough to sort rows per expert.
  // B200_ZV_TC=0 keeps every projection on linear.cu (A/B knob); fp32 models always do.
  int setup_tc() {
    const char* ev = getenv("B200_ZV_TC");
    use_tc = dt == DT_BF16 && !(ev && atoi(ev) == 0) && W % 8 == 0 && gemm_variant() == 2;
    if (!use_tc) return 0;
    int maxN = W;
    for (auto& s : spec) maxN = std::max(std::max(maxN, s.n_in), std::max(s.n_sh, 2 * s.ff));
    const size_t ws_bytes = std::max(gemm_workspace_bytes(env.sms), gemm_deferred_ws_bytes(env.sms));
    if (dalloc(&gemm_ws, ws_bytes)) return -3;
    const size_t n_counters = 2ull * (maxN / 128 + 2) * (env.Tcap / 32 + 2);
    if (dalloc(&gemm_counters, n_counters * sizeof(int))) return -3;
    const int bns[kGemmNumBlockN] = {32, 64, 128, 256, 512};
    for (int i = 0; i < kGemmNumBlockN; ++i)
      if (gemm_make_x_map(&xm_h[i], h, env.Tcap, W, W, bns[i])) { use_tc = false; return 0; }
    bool any_expert_tc = false;
    for (size_t i = 0; i < spec.size(); ++i) {
      const LayerSpec& s = spec[i];
      LayerWeights& w = wts[i];
      w.tc_in = gemm_plan_init(&w.p_in, w.w_in, s.n_in, W, W, gemm_ws, gemm_counters, env.sms) == 0;
      if (w.tc_in) w.p_in.ws_bytes = ws_bytes;
      w.tc_out = s.k_out % 8 == 0 && gemm_plan_init(&w.p_out, w.w_out, W, s.k_out, s.k_out, gemm_ws, gemm_counters, env.sms) == 0;
      for (int j = 0; j < kGemmNumBlockN && w.tc_out; ++j)
        if (gemm_make_x_map(&w.xm_out[j], ycat, env.Tcap, s.k_out, s.k_out, bns[j])) w.tc_out = false;
      if (w.tc_out) w.p_out.ws_bytes = ws_bytes;
      if (s.mlp && s.shared) {
        w.tc_shin = gemm_plan_init(&w.p_shin, w.sh_in, s.n_sh, W, W, gemm_ws, gemm_counters, env.sms) == 0;
        if (w.tc_shin) w.p_shin.ws_bytes = ws_bytes;
        w.tc_shdown = s.sff % 8 == 0 && gemm_plan_init(&w.p_shdown, w.sh_down, W, s.sff, s.sff, gemm_ws, gemm_counters, env.sms) == 0;
        for (int j = 0; j < kGemmNumBlockN && w.tc_shdown; ++j)
          if (gemm_make_x_map(&w.xm_shact[j], shact, env.Tcap, s.sff, s.sff, bns[j])) w.tc_shdown = false;
        if (w.tc_shdown) w.p_shdown.ws_bytes = ws_bytes;
      }
      if (s.mlp && s.ff % 8 == 0) {
        w.p_egu.resize(s.experts);
        w.p_edown.resize(s.experts);
        bool ok = true;
        for (int e = 0; e < s.experts && ok; ++e) {
          ok = gemm_plan_init(&w.p_egu[e], static_cast<bf16*>(w.e_gu) + static_cast<size_t>(e) * 2 * s.ff * W, 2 * s.ff, W, W, gemm_ws, gemm_counters, env.sms) == 0 &&
               gemm_plan_init(&w.p_edown[e], static_cast<bf16*>(w.e_down) + static_cast<size_t>(e) * W * s.ff, W, s.ff, s.ff, gemm_ws, gemm_counters, env.sms) == 0;
          w.p_egu[e].ws_bytes = w.p_edown[e].ws_bytes = ws_bytes;
        }
        if (!ok) { w.p_egu.clear(); w.p_edown.clear(); }
        else any_expert_tc = true;
      }
    }
    if (any_expert_tc) {
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
    for (size_t i = 0; i < spec.size(); ++i) {
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
      if (r != rows || c != cols) {
        *err = name + ": shape [" + std::to_string(r) + "," + std::to_string(c) + "] does not fit the config";
        return false;
      }
      return true;
    };
    int rc = 0;
#define MAT(name, dst, ld, row0, col0, rows, cols) do { if (!get(name, rows, cols)) return -4; rc |= put(dst, ld, row0, col0, v, rows, cols); } while (0)
#define VEC(name, dst, n) do { if (!get(name, 1, n)) return -4; rc |= putf(dst, v); } while (0)
    MAT("embed", embed, W, 0, 0, V, W);
    VEC("final.norm", fin_w, W);
    for (size_t i = 0; i < spec.size(); ++i) {
      const LayerSpec& s = spec[i];
      LayerWeights& w = wts[i];
      const std::string p = "l" + std::to_string(i) + ".", lf = p + "mix.left.", rt = p + "mix.right.", f = p + "mlp.";
      VEC(p + "norm1", w.norm1, W);
      MAT(lf + "q", w.w_in, W, s.off_lq, 0, s.l.heads * s.l.dim, W);
      MAT(lf + "k", w.w_in, W, s.off_lk, 0, s.l.kv_heads * s.l.dim, W);
      MAT(lf + "v", w.w_in, W, s.off_lv, 0, s.l.kv_heads * s.l.vdim, W);
      MAT(lf + "g", w.w_in, W, s.off_lg, 0, s.hv_l, W);
      MAT(rt + "q", w.w_in, W, s.off_rq, 0, s.r.heads * s.r.dim, W);
      MAT(rt + "k", w.w_in, W, s.off_rk, 0, s.r.heads * s.r.dim, W);
      MAT(rt + "v", w.w_in, W, s.off_rv, 0, s.hv_r, W);
      MAT(rt + "g", w.w_in, W, s.off_rg, 0, s.hv_r, W);
      MAT(lf + "o", w.w_out, s.k_out, 0, 0, W, s.hv_l);
      MAT(rt + "o", w.w_out, s.k_out, 0, s.hv_l, W, s.hv_r);
      VEC(rt + "norm", w.r_norm, s.hv_r);
      if (hyper) { VEC(p + "hc1.in", w.hc1.in, ns); VEC(p + "hc1.out", w.hc1.out, ns); if (!get(p + "hc1.mix", ns, ns)) return -4; rc |= putf(w.hc1.mix, v); }
      if (!s.mlp) continue;
      VEC(p + "norm2", w.norm2, W);
      if (hyper) { VEC(p + "hc2.in", w.hc2.in, ns); VEC(p + "hc2.out", w.hc2.out, ns); if (!get(p + "hc2.mix", ns, ns)) return -4; rc |= putf(w.hc2.mix, v); }
      MAT(f + "router", w.router, W, 0, 0, s.experts, W);
      for (int e = 0; e < s.experts; ++e) {
        const std::string ep = f + "e" + std::to_string(e) + ".";
        MAT(ep + "gate", w.e_gu, W, static_cast<size_t>(e) * 2 * s.ff, 0, s.ff, W);
        MAT(ep + "up", w.e_gu, W, static_cast<size_t>(e) * 2 * s.ff + s.ff, 0, s.ff, W);
        MAT(ep + "down", w.e_down, s.ff, static_cast<size_t>(e) * W, 0, W, s.ff);
      }
      if (s.shared) {
        MAT(f + "shared.gate", w.sh_in, W, 0, 0, s.sff, W);
        MAT(f + "shared.up", w.sh_in, W, s.sff, 0, s.sff, W);
        MAT(f + "shared.sg", w.router, W, s.experts, 0, 1, W);
        MAT(f + "shared.down", w.sh_down, s.sff, 0, 0, W, s.sff);
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
    uint64_t k = seed * 1000003ull + 29;
    auto M = [&](void* p, size_t n, float sc) { rc |= fill_uniform(p, dt, n, ++k, sc, 0.f, st); };
    auto F = [&](float* p, size_t n, float sc, float off) { if (p) rc |= fill_uniform(p, DT_F32, n, ++k, sc, off, st); };
    const float sw = 1.7f / sqrtf(static_cast<float>(W));
    M(embed, static_cast<size_t>(V) * W, 1.7f / sqrtf(static_cast<float>(W)));
    F(fin_w, W, 0.1f, 1.f);
    for (size_t i = 0; i < spec.size(); ++i) {
      const LayerSpec& s = spec[i];
      LayerWeights& w = wts[i];
      M(w.w_in, static_cast<size_t>(s.n_in) * W, sw);
      M(w.w_out, static_cast<size_t>(W) * s.k_out, 1.7f / sqrtf(static_cast<float>(s.k_out)));
      F(w.norm1, W, 0.1f, 1.f); F(w.r_norm, s.hv_r, 0.1f, 1.f);
      F(w.hc1.in, ns, 0.1f, 1.0f / ns); F(w.hc1.out, ns, 0.1f, 0.5f); F(w.hc1.mix, static_cast<size_t>(ns) * ns, 0.1f, 1.0f / ns);
      if (!s.mlp) continue;
      F(w.norm2, W, 0.1f, 1.f);
      F(w.hc2.in, ns, 0.1f, 1.0f / ns); F(w.hc2.out, ns, 0.1f, 0.5f); F(w.hc2.mix, static_cast<size_t>(ns) * ns, 0.1f, 1.0f / ns);
      M(w.router, static_cast<size_t>(s.experts + (s.shared ? 1 : 0)) * W, sw);
      M(w.e_gu, static_cast<size_t>(s.experts) * 2 * s.ff * W, sw);
      M(w.e_down, static_cast<size_t>(s.experts) * W * s.ff, 1.7f / sqrtf(static_cast<float>(s.ff)));
      if (s.shared) { M(w.sh_in, static_cast<size_t>(s.n_sh) * W, sw); M(w.sh_down, static_cast<size_t>(W) * s.sff, 1.7f / sqrtf(static_cast<float>(s.sff))); }
    }
    if (rc) return -2;
    return cudaStreamSynchronize(st) == cudaSuccess ? 0 : -2;
  }

  // ------------------------------------------------------------ forward
  int project(const GemmPlan& plan, bool tc, const CUtensorMap* xm, const void* X, const void* Wm, void* Y, int T, int N, int K) {
    if (tc) {
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
#define KRN(name, call) do { prof_start(); const int r_ = (call); if (r_ && !rc) { failed_kernel = name; failed_rc = r_; } rc |= r_; prof_stop(name); ++nl; } while (0)
  const char* failed_kernel = "";
  int failed_rc = 0;

  // the write-back of the last sublayer (y, its stream weights), still to be applied by the next stream kernel
  struct Pending {
    const void* y = nullptr;
    const Hyper* hc = nullptr;
  };
  HyperArgs boundary(const Pending& p, const float* in, const float* norm_w, void* out, DType to, const int* row_index, int rows) {
    HyperArgs a;
    a.x = x; a.streams = ns; a.stream_stride = xstride;
    a.y = p.y; a.ty = dt;
    a.mix = p.hc ? p.hc->mix : nullptr; a.out = p.hc ? p.hc->out : nullptr;
    a.in = in; a.norm_w = norm_w; a.eps = eps;
    a.h = out; a.th = to; a.row_index = row_index; a.rows = rows; a.W = W;
    return a;
  }

  int moe(const LayerSpec& s, const LayerWeights& w, int T, int64_t& nl) {
    cudaStream_t st = env.stream;
    int rc = 0;
    const int nr = s.experts + (s.shared ? 1 : 0);   // router logits and, behind them, the shared expert's gate logit
    KRN("moe_router", linear(linear_args(h, dt, w.router, dt, scores, DT_F32, T, nr, W), st));
    KRN("moe_route", moe_route(scores, topi, topw, T, s.experts, 1, 1, s.top, st, MOE_SIGMOID, nr));
    const void* shared_out = nullptr;
    const float* shared_gate = nullptr;
    if (s.shared) {
      KRN("shared_in", project(w.p_shin, w.tc_shin, xm_h, h, w.sh_in, sh, T, s.n_sh, W));
      KRN("glu", glu_clamped(sh, s.n_sh, shact, s.sff, dt, T, s.sff, s.slimit, 1.702f, st));
      KRN("shared_down", project(w.p_shdown, w.tc_shdown, w.xm_shact, shact, w.sh_down, sdown, T, W, s.sff));
      shared_out = sdown;
      shared_gate = scores + s.experts;
    }
    const long long gu_stride = 2ll * s.ff * W, down_stride = static_cast<long long>(W) * s.ff;
    static const int moe_tc_min = [] { const char* e = getenv("B200_ZV_MOE_TC_MIN_T"); return e ? atoi(e) : 256; }();   // A/B knob
    const bool per_expert = !w.p_egu.empty() && T >= moe_tc_min;
    if (T * s.top <= 64) {
      // decode-sized steps: one weight-streaming pass per chosen (token, expert) pair, rows in pair order
      LinearArgs up = linear_args(h, dt, w.e_gu, dt, egu, dt, T * s.top, 2 * s.ff, W);
      up.wbs = gu_stride; up.row_scale = topw;
      const PickedRows pu = {T * s.top, nullptr, s.top, iota, topi};
      KRN("moe_up", linear_picked_rows(up, pu, st));
      KRN("glu", glu_clamped(egu, 2 * s.ff, eact, s.ff, dt, T * s.top, s.ff, s.limit, 1.702f, st));
      LinearArgs dn = linear_args(eact, dt, w.e_down, dt, edown, DT_F32, T * s.top, W, s.ff);
      dn.wbs = down_stride;
      const PickedRows pd = {T * s.top, iota, 1, iota, topi};
      KRN("moe_down", linear_picked_rows(dn, pd, st));
      // pair p of token t is row t * top + k: the combine walks them through an identity table
      KRN("moe_combine", combine_identity(T, s.top, shared_out, shared_gate, nr, st));
      return rc;
    }
    const int cap = (T * s.top + 63) / 64 * 64 + s.experts * 64;
    KRN("moe_align", moe_align(topi, T, s.top, s.experts, sorted_rows, tile_group, pair_pos, cap, st, per_expert ? expert_rows : nullptr, topw, sorted_w));
    if (per_expert) {
      // Large steps: every expert's rows are one tcgen05 GEMM.  The row counts come back to the host (one small copy and a
      // wait per layer, paid only by steps of hundreds of tokens); the inputs are gathered into sorted order, scaled by
      // their router weight in fp32 and rounded once.
      KRN("moe_gather", moe_gather_bf16(h, sorted_rows, hsorted, cap, W, st, sorted_w));
      if (cudaMemcpyAsync(expert_rows_host, expert_rows, static_cast<size_t>(s.experts) * 2 * sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
          cudaStreamSynchronize(st) != cudaSuccess) rc = -2;
      prof_start();
      for (int e = 0; e < s.experts && !rc; ++e) {
        const int start = expert_rows_host[2 * e], cnt = expert_rows_host[2 * e + 1];
        if (cnt <= 0) continue;
        const int bn = gemm_block_n_for(cnt);
        CUtensorMap tm;
        if (gemm_make_x_map(&tm, static_cast<bf16*>(hsorted) + static_cast<size_t>(start) * W, cnt, W, W, bn)) { rc = -2; break; }
        rc |= gemm_run(w.p_egu[e], tm, bn, static_cast<bf16*>(egu) + static_cast<size_t>(start) * 2 * s.ff, 2 * s.ff, cnt, st);
        ++nl;
      }
      prof_stop("moe_up");
      KRN("glu", glu_clamped(egu, 2 * s.ff, eact, s.ff, dt, cap, s.ff, s.limit, 1.702f, st));
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
      KRN("moe_combine", moe_combine_add(edown16, DT_BF16, pair_pos, nullptr, shared_out, shared_gate, nr, fo, dt, T, s.top, W, st));
      return rc;
    }
    LinearArgs up = linear_args(h, dt, w.e_gu, dt, egu, dt, cap, 2 * s.ff, W);
    up.x_rows = sorted_rows; up.tile_group = tile_group; up.wbs = gu_stride; up.row_scale = sorted_w;
    KRN("moe_up", linear(up, st));
    KRN("glu", glu_clamped(egu, 2 * s.ff, eact, s.ff, dt, cap, s.ff, s.limit, 1.702f, st));
    LinearArgs dn = linear_args(eact, dt, w.e_down, dt, edown, DT_F32, cap, W, s.ff);
    dn.tile_group = tile_group; dn.wbs = down_stride;
    KRN("moe_down", linear(dn, st));
    KRN("moe_combine", moe_combine_add(edown, DT_F32, pair_pos, nullptr, shared_out, shared_gate, nr, fo, dt, T, s.top, W, st));
    return rc;
  }
  int combine_identity(int T, int top, const void* shared_out, const float* shared_gate, int ld_gate, cudaStream_t st) {
    return moe_combine_add(edown, DT_F32, iota, nullptr, shared_out, shared_gate, ld_gate, fo, dt, T, top, W, st);
  }

  int forward(const StepBatch& b, int* sampled, float* host_logits, int64_t* launches) override {
    cudaStream_t st = env.stream;
    const int T = b.T;
    int rc = 0;
    int64_t nl = 0;
    const size_t es = dtype_bytes(dt);
    auto col = [&](void* base, size_t off) { return static_cast<void*>(static_cast<uint8_t*>(base) + off * es); };
    KRN("embed", embed_scaled(embed, dt, b.ids, x, T, W, V, emb_scale, ns, xstride, st));
    Pending pend;
    for (size_t ri = 0; ri < run.size() && !rc; ++ri) {
      const LayerRun& r = run[ri];
      const LayerSpec& s = spec[r.layer];
      const LayerWeights& w = wts[r.layer];
      KRN("stream_norm", hyper_step(boundary(pend, w.hc1.in, w.norm1, h, dt, nullptr, T), st));
      KRN("proj_in", project(w.p_in, w.tc_in, xm_h, h, w.w_in, inb, T, s.n_in, W));
      QkPrepArgs qp;
      qp.q = col(inb, s.off_lq); qp.k = col(inb, s.off_lk); qp.v = col(inb, s.off_lv); qp.ld = s.n_in; qp.t = dt;
      qp.rope = w.rope; qp.rot_dims = s.l.rot_dims; qp.unit_norm = true; qp.eps = eps;
      qp.positions = b.pos; qp.slots = b.slots; qp.qn = qn; qp.cache = r.cache;
      qp.T = T; qp.heads = s.l.heads; qp.kv_heads = s.l.kv_heads; qp.dim = s.l.dim; qp.vdim = s.l.vdim;
      KRN("qk_prep", qk_rope_norm_cache(qp, st));
      WindowAttnArgs wa;
      wa.qn = qn; wa.cache = r.cache; wa.t = dt; wa.positions = b.pos; wa.seq_of_tok = b.seq_of_tok; wa.block_tables = b.btab;
      wa.max_blocks = b.max_blocks; wa.page = env.page;
      wa.gate = col(inb, s.off_lg); wa.ldg = s.n_in; wa.out_scale = s.left_scale; wa.y = ycat; wa.ldy = s.k_out;
      wa.T = T; wa.heads = s.l.heads; wa.kv_heads = s.l.kv_heads; wa.dim = s.l.dim; wa.vdim = s.l.vdim;
      wa.window = std::min(s.l.window, env.max_model_len); wa.keep_first = std::min(s.l.keep_first, env.max_model_len); wa.scale = s.l.scale;
      wa.seqs = b.seqs; wa.nseq = b.nseq; wa.max_ctx = b.max_ctx;
      KRN("window_attention", window_attention(wa, st));
      GlaArgs g;
      g.qkv = inb; g.t = dt; g.ld = s.n_in; g.q_off = s.off_rq; g.k_off = s.off_rk; g.v_off = s.off_rv;
      g.z = nullptr; g.z_bias = nullptr; g.inv_tau = 1.f; g.q_scale = 1.f; g.T = T;
      g.states = r.state; g.seqs = b.seqs; g.nseq = b.nseq;
      g.heads = s.r.heads; g.dim = s.r.dim; g.vdim = s.r.vdim; g.o = o32;
      g.head_decay = w.decay; g.act = GLA_ACT_SILU;
      KRN("lightning_scan", gla_scan(g, st));
      OutGateArgs og;
      og.o = o32; og.g = col(inb, s.off_rg); og.ldg = s.n_in; og.w = w.r_norm; og.eps = eps;
      og.y = col(ycat, s.hv_l); og.ldy = s.k_out; og.t = dt; og.T = T; og.heads = s.r.heads; og.vdim = s.r.vdim;
      og.joint = true; og.gate_act = GATE_SIGMOID; og.out_scale = s.right_scale;
      KRN("lightning_out_gate", recurrent_out_gate(og, st));
      KRN("proj_out", project(w.p_out, w.tc_out, w.xm_out, ycat, w.w_out, ao, T, W, s.k_out));
      pend.y = ao; pend.hc = hyper ? &w.hc1 : nullptr;
      if (s.mlp) {
        KRN("stream_norm", hyper_step(boundary(pend, w.hc2.in, w.norm2, h, dt, nullptr, T), st));
        rc |= moe(s, w, T, nl);
        pend.y = fo; pend.hc = hyper ? &w.hc2 : nullptr;
      }
      if (residual_sink && !rc) {
        // debug: apply the write-back now and read the sum of the streams
        if (!sumbuf && dalloc(&sumbuf, static_cast<size_t>(env.Tcap) * W * sizeof(float))) rc = -3;
        KRN("stream_norm", hyper_step(boundary(pend, nullptr, nullptr, sumbuf, DT_F32, nullptr, T), st));
        pend = Pending();
        const size_t at = residual_sink->size();
        residual_sink->resize(at + static_cast<size_t>(T) * W);
        if (rc || cudaMemcpyAsync(residual_sink->data() + at, sumbuf, static_cast<size_t>(T) * W * sizeof(float), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess) rc = -2;
      }
    }
    if (pend.y) KRN("stream_norm", hyper_step(boundary(pend, nullptr, nullptr, nullptr, dt, nullptr, T), st));
    // head: RMS norm of the summed streams of the wanted rows, logits against the embedding table in fp32, greedy choice
    for (int r0 = 0; r0 < b.S && !rc; r0 += row_cap) {
      const int n = std::min(row_cap, b.S - r0);
      KRN("stream_norm", hyper_step(boundary(Pending(), nullptr, fin_w, hrow, dt, b.rows + r0, n), st));
      KRN("head", linear(linear_args(hrow, dt, embed, dt, logits, DT_F32, n, V, W), st));
      KRN("argmax", argmax_f32(logits, sampled + r0, n, V, st));
      if (host_logits && cudaMemcpyAsync(host_logits + static_cast<size_t>(r0) * V, logits, static_cast<size_t>(n) * V * sizeof(float),
                                         cudaMemcpyDeviceToHost, st) != cudaSuccess) rc = -2;
    }
    if (launches) *launches += nl;
    if (rc) { set_error("Zinavik forward: %s failed with %d (%s)", failed_kernel, failed_rc, cudaGetErrorString(cudaGetLastError())); return -2; }
    return 0;
  }
};

}  // namespace

#undef KRN

std::unique_ptr<Model> make_zinavik(const JVal& config, DType dtype, std::string* err) {
  std::unique_ptr<Zinavik> m(new Zinavik(dtype));
  if (!m->parse(config, err)) return nullptr;
  return std::unique_ptr<Model>(m.release());
}

}  // namespace b200
