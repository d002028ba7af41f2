// C++ host of the decoder designs whose checkpoint configuration lists the layers one by one (Vamadra, Risolorn, Nagosun, Goguzen), on an
// fp32 residual stream.  A layer is a mixer plus an optional feed-forward, put together in one of four block forms:
//   block 0  sequential sublayers with the norm on each sublayer's OUTPUT:  x += norm(mixer(x));  x += norm(ff(x))
//   block 1  parallel sublayers under one Dynamic-Tanh pre-norm:            h = dyt(x);  x += mixer(h) + ff(h)
//   block 2  "sandwich": a grouped RMS norm before AND after each sublayer, the sublayer's result gated by a logistic
//            projection of its input, the sum scaled:  h = gn(x); x += m * gn(f(h) * logistic(W_rg h + b))   (mixers 0 and 1)
//   block 3  pre-norm sequential sublayers with plain-weight RMS norms:      x += mixer(rms(x) w1);  x += ff(rms(x) w2)   (mixers 1 and 4);
//            a layer may run with another layer's weights (and a cache / state of its own); logits are scaled and soft-capped
// Mixers: 0 latent attention (compressed paged cache, shared rotated key part, per-head sink, logistic output gate, optional
// reuse of an earlier layer's cache); 1 grouped-query attention with biases, rotary embedding from a frequency table, a
// chunk-local causal mask and a sink, over a paged K/V cache (block 2 adds: sliding window, score soft cap, linear distance
// bias, unit-RMS cached values, a sink of score zero, an element-wise output gate); 2 gated delta rule behind short causal
// convolutions; 3 xLSTM matrix memory; 4 two branches side by side on the same input -- grouped-query attention and a state-space layer
// (scalar decay per head, short causal convolution, gated group-normed read-out) -- each branch's result RMS-normed over the width, the
// mixer's result their mean.  Block 3 gives the attention (mixer 1 and the attention branch of 4) further options: RMS norm of q and k per
// head or over the whole projection, a query factor that grows with the logarithm of the position, values that are the keys as projected,
// a window that keeps the first positions visible, rotary frequencies rescaled by wavelength.  Mixers 2, 3 and 4 keep an fp32 state per
// request in numbered state slots.  Feed-forward: dense SwiGLU or a mixture of experts (softmax or logistic router or plain top logits;
// relu^2, gated-SiLU or clamped gated experts; a shared expert with or without a gate).
//
// Same structure as the other hosts in this folder: kernels are reached only through the C ABI
// (include/pegainfer_kernels.h) resolved with dlopen; paging reuses pq::PagePool / pq::KvState; a step is planned and
// validated first and committed last; one packed metadata block per step is uploaded with a single copy.
//
// One entry point runs everything: step() takes a ragged batch -- for each live request its next tokens, whether that
// is a portion of a prompt or one decoded token -- appends to the cache, advances the recurrent state and returns logits
// for the rows asked for.  Element type of weights / activations / cache is bf16 (tensor-core GEMMs of this library) or
// float (plain FMA kernels, no reduced-precision matrix mode); softmax, norms, routers, recurrences and the residual sum
// are fp32 in both.
#include <dlfcn.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <set>
#include <string>
#include <tuple>

#include "qwen3_host.hpp"

namespace pv {

using pq::DeviceBuf;

struct LayerCfg {  // mirrored by ctypes in pegainfer_b200/vamadra.py
  int heads, dim, rot_dim, vdim, kv_rank, kv_from;  // kv_from < 0: the layer owns its cache
  int rot_dims;                                      // rotated entries of the rot_dim slice
  float rot_base, scale;
  int has_scaling;
  float s_factor, s_original, s_fast, s_slow;  // YaRN
  int mlp_kind;                                // 0 none, 1 dense (SwiGLU), 2 mixture of experts
  int ff;                                      // dense: hidden size
  int experts, top, groups, keep;
  float route_scale;
  int expert_ff, shared_ff;  // shared_ff 0: no shared expert
  // mixers 1-3 (mixer_kind 0 = latent attention uses the fields above only)
  int mixer_kind;            // 0 latent attention, 1 grouped-query attention, 2 gated delta rule, 3 xLSTM matrix memory
  int kv_heads;              // key/value heads (1, 2); query/key heads of the delta rule
  int chunk;                 // 1: chunk-local causal mask of this size, 0 = plain causal
  int conv;                  // 2: taps of the short convolutions
  int rot_interleaved;       // 1: rotary pairs (2i, 2i+1) instead of (i, i + dims/2)
  float gate_cap;            // 3: soft cap of the log gates
  int router_kind;           // 0 softmax scores, best expert per group, renormalised; 1 logistic scores + choice correction, two best per group, plain
  int expert_act;            // 0 relu^2, 1 gated SiLU
  // options read by block 2 (all off when zero)
  int window;                // attention (0, 1): a query at position p sees keys p - window + 1 .. p
  float softcap;             // 1: scaled score <- softcap * tanh(score / softcap)
  float slope_log2;          // 1: head h subtracts 2^(-slope_log2 (h + 1) / heads) * distance from the score
  int value_norm;            // 1: cached values are divided by their root mean square per head (eps of the model, no weight)
  int sink_kind;             // 0 learned per-head sink 'mix.sink', 1 none, 2 a sink of score zero (one added to the softmax denominator)
  int out_gate;              // 1: 1 = heads' outputs times logistic(W_g h) element by element ('mix.g' [heads * vdim, width])
  int proj_bias;             // 1: q, k, v and o projections carry biases ('.b')
  // options read by block 3 (all off when zero)
  int keep_first;            // attention with a window: the first keep_first positions stay visible
  int qk_norm;               // 1: RMS norm of q and k per head, weights 'q.norm' / 'k.norm' [dim]; 2: over the whole projection, weights [heads*dim] / [kv_heads*dim]
  float q_temp_coef;         // q *= 1 + q_temp_coef * ln(floor((p + 1) / q_temp_every) + 1)
  int q_temp_every;
  int values_are_keys;       // 1: no value projection, a head's values are its keys as projected
  int scaling_kind;          // rotary scaling (has_scaling): 0 YaRN ramp over the pair index; 1 by wavelength: s_fast = 'high', s_slow = 'low'
  int ssm_heads, ssm_vdim, ssm_state, ssm_groups, ssm_norm_groups;  // mixer 4, state-space branch (taps in `conv`)
  float act_limit, act_slope;  // expert_act 2: g = min(gate, limit), u = clamp(up, +-limit), g logistic(slope g) (u + 1)
  float shared_limit;        // the shared expert's limit (router_kind 2: shared expert of the same form, no gate)
  int weights_of;            // >= 0: the layer runs with that layer's weights
};
struct ModelCfg {
  int vocab, width, n_layers;
  float eps;
  int f32, page_size, num_pages, max_requests, device, enable_pdl;
  int block_kind;  // 0 sequential sublayers, offset RMS norm on their outputs; 1 parallel sublayers under a Dynamic-Tanh pre-norm; 2 sandwich
  float embed_scale, logit_scale;
  int norm_groups;        // block 2: parts of a row that are normed separately
  float residual_mult;    // block 2: multiplier of every sublayer's normed result
  int gated_residual;     // block 2: sublayer results times logistic(W_rg h + b) ('rg1' / 'rg2') before their norm
  float logit_softcap;    // block 3: logits <- cap * tanh(logits / cap) after the multiplier (0: none)
};

struct Lib {
  void* handle = nullptr;
  // every design / the block forms that route to experts / the ones with a dense feed-forward / one block form each
#define PV_COMMON(X)                                                                                                                       \
  X(cuda_set_device) X(cublas_init) X(cublas_destroy) X(gemm_cuda) X(flashinfer_top1_cuda) X(pk_b200_set_pdl) X(pk_b200_launch_count)      \
  X(pk_res32_skinny_proj) X(pk_convert) X(pk_gemm_strided) X(pk_proj_rows_f32out) X(pk_scale_to_f32) X(pk_top1_rows_f32)
#define PV_MOE(X) X(pk_moe_down_combine) X(pk_moe_grouped_workspace_bytes) X(pk_moe_up_act_p) X(pk_moe_grouped_act_p)
#define PV_DENSE(X) X(pk_act) X(pk_b200_gemv_fused) X(pk_b200_gemm_swiglu)
#define PV_BLOCK0(X)                                                                                                                        \
  X(pk_res32_embed) X(pk_res32_offset_norm_add) X(pk_res32_offset_norm_rows) X(pk_rope_slice) X(pk_latent_kv_append) X(pk_latent_attention) \
  X(pk_router_grouped_topk)
#define PV_BLOCK1(X)                                                                                                                        \
  X(pk_res32_embed_scaled) X(pk_res32_add_dyt) X(pk_res32_dyt_rows) X(pk_gqa_rope_append) X(pk_gqa_attention) X(pk_causal_conv_silu)       \
  X(pk_gated_delta_seq) X(pk_mlstm_seq) X(pk_router_topk_ex)
#define PV_BLOCK13(X) X(pk_head_norm_gate)
#define PV_BLOCK23(X) X(pk_res32_gnorm_rows) X(pk_gqa_attention_ex)
#define PV_BLOCK3(X)                                                                                                                        \
  X(pk_res32_embed_scaled_norm) X(pk_res32_branches_add_norm) X(pk_logits_scale_cap) X(pk_act_clamped) X(pk_gqa_norm_append)               \
  X(pk_causal_conv_silu_bias) X(pk_ssd_seq) X(pk_router_topk_logits)
#define PV_BLOCK2(X)                                                                                                                        \
  X(pk_res32_embed_gnorm) X(pk_res32_gated_gnorm_add) X(pk_gqa_rope_append_ex) X(pk_rope_slice_ex)   \
  X(pk_latent_kv_append_ex) X(pk_latent_attention_ex) X(pk_b200_gemm_segments)
#define PV_FN(name) decltype(&::name) name = nullptr;
  PV_COMMON(PV_FN) PV_MOE(PV_FN) PV_DENSE(PV_FN) PV_BLOCK0(PV_FN) PV_BLOCK1(PV_FN) PV_BLOCK2(PV_FN) PV_BLOCK13(PV_FN) PV_BLOCK23(PV_FN) PV_BLOCK3(PV_FN)
#undef PV_FN
  // a library built for one design need not hold the other block form's kernels: only what `block_kind` runs is required
  std::string load(const std::string& p, int block_kind) {
    handle = dlopen(p.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!handle) return std::string("dlopen failed: ") + dlerror();
    std::string missing;
#define PV_REQ(name)                                             \
  name = reinterpret_cast<decltype(name)>(dlsym(handle, #name)); \
  if (!name) missing += std::string(" ") + #name;
    PV_COMMON(PV_REQ)
    if (block_kind == 0) {
      PV_MOE(PV_REQ) PV_DENSE(PV_REQ) PV_BLOCK0(PV_REQ)
    } else if (block_kind == 1) {
      PV_MOE(PV_REQ) PV_BLOCK1(PV_REQ) PV_BLOCK13(PV_REQ)
    } else if (block_kind == 2) {  // the sandwich block form has no mixture of experts
      PV_DENSE(PV_REQ) PV_BLOCK2(PV_REQ) PV_BLOCK23(PV_REQ)
    } else {
      PV_MOE(PV_REQ) PV_BLOCK3(PV_REQ) PV_BLOCK13(PV_REQ) PV_BLOCK23(PV_REQ)
    }
#undef PV_REQ
    return missing.empty() ? "" : "kernel library " + p + " lacks:" + missing;
  }
  ~Lib() {
    if (handle) dlclose(handle);
  }
};

static const int kGraphCtxBucket = 512;   // captured decode steps are keyed by the context length rounded up to this
static const int kGroupedMinTokens = 32;  // from this many tokens in a step the experts run bucketed

struct Mat {
  DeviceBuf d;
  int rows = 0, cols = 0;
};
struct Layer {
  LayerCfg c{};
  Mat norm1, norm2, q, dkv, dkv_norm, uk, uk_t, uv, sink, g, o;  // mixer; uk_t = W_uk per head as [rank, dim] (made at load)
  Mat gate_up, down;                                       // dense: [gate ; up] stacked
  Mat e_up, e_down, router, s_up, s_down, s_gate;          // experts stacked [experts * ff, width] / [experts * width, ff]
  // mixers 1-3 / block 1: stacked projections [q | k | v (| gate)], their bias, the few-row fp32 projections [router | za | zb]
  Mat nb, qkv, qkv_bias, small, conv_w, hnorm;
  Mat norm1b, norm2b, o_bias, rg1_bias, rg2, rg2_bias;    // block 2: post-norms, output bias, gates of the sublayer results (rg1 is stacked into qkv)
  DeviceBuf alpha32, corr32, p0_32, p1_32, p2_32;          // float copies of small parameter vectors (made in finalize)
  Mat alpha, corr, p0, p1, p2;
  Mat qn, kn, conv_b, o2, lout, rout;                      // block 3: q / k norm weights; mixer 4: convolution bias, second output projection, branch norms
  int wsrc = 0;                                            // the layer whose weights this layer runs with (itself unless the configuration says otherwise)
  int64_t state_off = 0;                                   // float offset of the layer's block inside a state slot
  DeviceBuf freq;                                          // [rot_dims / 2] fp32 angular frequencies
  float mag = 1.f;
  int owner = -1;       // layer whose cache this layer reads (itself when it owns one)
  int64_t cache_off = 0;  // element offset of the owner's block inside a page
  std::set<std::string> got;
};

struct Model {
  Lib k;
  ModelCfg c{};
  std::vector<Layer> layers;
  std::string err;
  cudaStream_t st = nullptr;
  int es = 2;  // element size
  Mat embed, head, final_norm, final_b, final_alpha;
  DeviceBuf final_alpha32;
  Mat embed_norm;                // block 2: norm of the embedding
  DeviceBuf zero_sink;           // block 2: [heads] zeros, the sink of score zero
  DeviceBuf rgbuf;               // block 2: gate pre-activations [tokens, width]
  DeviceBuf cache, state;        // paged cache pool; recurrent state, one slot per request id
  int64_t slot_stride = 0;       // floats per state slot
  std::vector<char> fresh;       // request slot allocated and not stepped yet: its state is zeroed before the first step
  int64_t page_stride = 0;
  pq::PagePool pool;
  std::vector<pq::KvState> reqs;
  bool finalized = false;
  // per-step scratch, grown to the largest step seen
  int cap_t = 0, cap_r = 0;
  DeviceBuf h32, big, convo, zs, orec, den;  // block 1: unrounded norm output, stacked projections, conv outputs, few-row fp32, read-out
  DeviceBuf ao2, mix2;                       // mixer 4: the state-space branch's gated read-out and its projection
  DeviceBuf x, xa, q, dkv, qa, gate, olat, ao, mix, gu, act, z, ids, wts, hid, yf, sgl, sh, xr, logits_e, logits_f, logits_bf, sampled_d, top1_val,
      top1_states, trail, moe_ws;
  DeviceBuf meta_d;
  int* meta_h = nullptr;
  size_t meta_cap = 0;
  int* sampled_h = nullptr;
  int pages_at = 0;  // int offset of the page lists inside the step's metadata block
  bool keep_trail = false;
  int trail_tokens = 0;
  // captured decode steps
  typedef std::tuple<int, int, int, int> GraphKey;  // entries, logits rows, sampling, context bucket
  std::map<GraphKey, cudaGraphExec_t> graphs;
  std::set<GraphKey> seen;
  bool use_graph = true;
  // widest layer
  int mx_big = 0, mx_conv = 0, mx_small = 0, mx_inner = 0;
  int mx_q = 0, mx_dkv = 0, mx_qa = 0, mx_h = 0, mx_olat = 0, mx_ao = 0, mx_gu = 0, mx_act = 0, mx_e = 0, mx_top = 0, mx_hid = 0;

  bool fail(const std::string& m) {
    err = m;
    return false;
  }
  bool cu(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return true;
    err = std::string(what) + ": " + cudaGetErrorString(e);
    return false;
  }
  bool rc(int r, const char* what) {
    if (r == 0) return true;
    err = std::string(what) + " failed (" + (r > 0 ? cudaGetErrorString((cudaError_t)r) : r == -1 ? "invalid argument" : "shape out of range") + ")";
    return false;
  }
  ~Model() {
    if (st) cudaStreamSynchronize(st);
    drop_graphs();
    if (meta_h) cudaFreeHost(meta_h);
    if (sampled_h) cudaFreeHost(sampled_h);
    if (k.cublas_destroy) k.cublas_destroy();
    if (st) cudaStreamDestroy(st);
  }
  bool configure(const ModelCfg& mc, const LayerCfg* lc);
  bool put(Mat& m, int rows, int cols, int row0, const void* src, int src_rows, const std::string& name, int got_rows, int got_cols);
  bool load_tensor(const std::string& name, const void* data, int rows, int cols, int is_f32);
  bool finalize();
  bool ensure_scratch(int T, int R);
  bool lin(const Mat& W, const void* X, void* Y, int N);
  bool skinny(const Mat& W, float* out, int T, const char* what, const float* in32 = nullptr);
  bool put_rows(Mat& m, int rows, int cols, int row0, int row_step, const void* src, int src_rows, const std::string& name, int got_rows, int got_cols);
  bool to_f32(const Mat& m, DeviceBuf* out);
  bool put_uk(Layer& L, const void* data, const std::string& name, int rows, int cols);
  bool run_experts(const Layer& L, int T, const void* shared, const float* shared_gate);
  bool run_prenorm_layer(int li, int T, int max_kv, const int* M, int n);
  bool run_parallel_layer(int li, int T, const int* M, int n);
  bool run_sandwich_layer(int li, int T, int max_kv, const int* M);
  bool lin_segments(const Mat& W, const void* X, void* const* Y, const int* seg_rows, int N);
  bool run_layer(int li, int T, int max_kv, const int* d_pos, const int* d_req, const int* d_poff, const int* d_pages);
  bool forward(int T, int n, int n_rows, int max_kv, int want_sample);
  bool step(int n, const int* tokens, const int* lens, const int* rids, int n_rows, const int* rows, int want_sample);
  void drop_graphs() {
    for (auto& g : graphs)
      if (g.second) cudaGraphExecDestroy(g.second);
    graphs.clear();
    seen.clear();
  }
};

static std::string lname(int i, const char* s) { return "l" + std::to_string(i) + "." + s; }

bool Model::configure(const ModelCfg& mc, const LayerCfg* lc) {
  c = mc;
  es = c.f32 ? 4 : 2;
  if (c.vocab <= 0 || c.width <= 0 || c.n_layers <= 0) return fail("vocab, width and the number of layers must be positive");
  if (c.block_kind < 0 || c.block_kind > 3) return fail("unknown block form");
  if (c.block_kind == 3 && c.logit_softcap < 0.f) return fail("logit_softcap must not be negative");
  if (c.block_kind == 2 && (c.norm_groups <= 0 || c.width % c.norm_groups)) return fail("norm.groups must divide the width");
  if (c.page_size <= 0) c.page_size = 16;
  if (c.max_requests <= 0) c.max_requests = 4;
  layers.resize(c.n_layers);
  int64_t off = 0, soff = 0;
  for (int i = 0; i < c.n_layers; ++i) {
    Layer& L = layers[i];
    L.c = lc[i];
    const LayerCfg& a = L.c;
    if (a.mixer_kind < 0 || a.mixer_kind > 4) return fail(lname(i, "mixer: unknown kind"));
    if (c.block_kind == 3 ? (a.mixer_kind != 1 && a.mixer_kind != 4)
                          : a.mixer_kind == 4 || (c.block_kind == 2 ? a.mixer_kind > 1 : (a.mixer_kind == 0) != (c.block_kind == 0)))
      return fail(lname(i, "mixer: not available in this block form"));
    L.wsrc = i;
    if (c.block_kind == 3 && a.weights_of >= 0) {
      if (a.weights_of >= c.n_layers || lc[a.weights_of].weights_of >= 0) return fail(lname(i, "weights_of must name a layer with weights of its own"));
      const LayerCfg& o = lc[a.weights_of];
      if (o.mixer_kind != a.mixer_kind || o.heads != a.heads || o.kv_heads != a.kv_heads || o.dim != a.dim || o.vdim != a.vdim || o.mlp_kind != a.mlp_kind ||
          o.experts != a.experts || o.expert_ff != a.expert_ff || o.shared_ff != a.shared_ff || o.ssm_heads != a.ssm_heads || o.ssm_vdim != a.ssm_vdim ||
          o.ssm_state != a.ssm_state || o.ssm_groups != a.ssm_groups || o.conv != a.conv || o.qk_norm != a.qk_norm)
        return fail(lname(i, "sizes differ from the layer whose weights it uses"));
      L.wsrc = a.weights_of;
    }
    if (a.window < 0 || a.softcap < 0.f || a.slope_log2 < 0.f) return fail(lname(i, "mixer: mask.size, softcap and the bias slope must not be negative"));
    if (a.heads <= 0 || a.dim <= 0 || a.vdim <= 0) return fail(lname(i, "mixer: sizes must be positive"));
    if (a.mixer_kind == 0) {
      if (a.kv_rank <= 0 || a.rot_dim < 0) return fail(lname(i, "mixer: sizes must be positive"));
      if (a.rot_dims < 0 || a.rot_dims > a.rot_dim || (a.rot_dims & 1)) return fail(lname(i, "mixer: rot.dims must be even and at most rot_dim"));
      if (a.kv_rank > 1024) return fail(lname(i, "mixer: kv_rank above 1024 is outside the attention kernel's range"));
      if (a.kv_from >= 0) {
        if (a.kv_from >= i || layers[a.kv_from].c.kv_from >= 0) return fail(lname(i, "mixer: kv_from must name an earlier layer that owns a cache"));
        const LayerCfg& o = layers[a.kv_from].c;
        if (o.kv_rank != a.kv_rank || o.rot_dim != a.rot_dim) return fail(lname(i, "mixer: kv_rank / rot_dim differ from the layer it borrows from"));
        L.owner = a.kv_from;
        L.cache_off = layers[a.kv_from].cache_off;
      } else {
        L.owner = i;
        L.cache_off = off;
        off += (int64_t)c.page_size * (a.kv_rank + a.rot_dim);
      }
      mx_q = std::max(mx_q, a.heads * (a.dim + a.rot_dim));
      mx_dkv = std::max(mx_dkv, a.kv_rank + a.rot_dim);
      mx_qa = std::max(mx_qa, a.heads * (a.kv_rank + a.rot_dim));
      mx_olat = std::max(mx_olat, a.heads * a.kv_rank);
    } else {
      if (a.kv_heads <= 0 || a.heads % a.kv_heads) return fail(lname(i, "mixer: heads must be a multiple of kv_heads"));
      if (a.dim > 256 || a.vdim > 256) return fail(lname(i, "mixer: head sizes above 256 are outside the kernels' range"));
      const int nqk = (a.mixer_kind == 1 || a.mixer_kind == 4) ? a.heads * a.dim + a.kv_heads * a.dim : 2 * a.kv_heads * a.dim;
      if (a.mixer_kind == 4) {
        if (a.ssm_heads <= 0 || a.ssm_vdim <= 0 || a.ssm_state <= 0 || a.ssm_groups <= 0 || a.ssm_heads % a.ssm_groups || a.conv <= 0 ||
            a.ssm_norm_groups <= 0 || (a.ssm_heads * a.ssm_vdim) % a.ssm_norm_groups)
          return fail(lname(i, "mixer: inconsistent state-space branch"));
        if (a.ssm_state > 256) return fail(lname(i, "mixer: state sizes above 256 are outside the kernels' range"));
        if (!a.values_are_keys || a.dim != a.vdim) return fail(lname(i, "mixer: the attention branch caches its keys as values (vdim must equal dim)"));
        const int inner = a.ssm_heads * a.ssm_vdim, C = inner + 2 * a.ssm_groups * a.ssm_state;
        L.state_off = soff;
        soff += (int64_t)a.ssm_heads * a.ssm_state * a.ssm_vdim + (int64_t)(a.conv - 1) * C;
        mx_conv = std::max(mx_conv, C);
        mx_inner = std::max(mx_inner, inner);
      }
      if (c.block_kind == 3) {
        if (a.qk_norm < 0 || a.qk_norm > 2 || a.q_temp_every < 0 || a.keep_first < 0) return fail(lname(i, "mixer: inconsistent attention options"));
        if (a.values_are_keys && a.dim != a.vdim) return fail(lname(i, "mixer: values that are keys need vdim == dim"));
      }
      if (a.mixer_kind == 1 || a.mixer_kind == 4) {
        if (a.rot_dims < 0 || a.rot_dims > a.dim || (a.rot_dims & 1)) return fail(lname(i, "mixer: rot.dims must be even and at most dim"));
        if (a.chunk < 0) return fail(lname(i, "mixer: mask.size must be positive"));
        L.owner = i;
        L.cache_off = off;
        off += (int64_t)c.page_size * a.kv_heads * (a.dim + a.vdim);
        off = (off + 7) / 8 * 8;  // every layer's block starts 16-byte aligned in both element types
        mx_big = std::max(mx_big, nqk + a.kv_heads * a.vdim + (c.block_kind == 2 ? (a.out_gate ? a.heads * a.vdim : 0) + (c.gated_residual ? c.width : 0) : 0));
        if (a.mixer_kind == 4) mx_big = std::max(mx_big, nqk + 2 * a.ssm_heads * a.ssm_vdim + 2 * a.ssm_groups * a.ssm_state + a.ssm_heads);
        mx_q = std::max(mx_q, a.heads * a.dim);
      } else {
        if (a.mixer_kind == 2 && a.conv <= 0) return fail(lname(i, "mixer: conv must be positive"));
        if (a.mixer_kind == 3 && (a.kv_heads != a.heads || !(a.gate_cap > 0.f))) return fail(lname(i, "mixer: inconsistent matrix memory"));
        L.state_off = soff;
        soff += (int64_t)a.heads * a.dim * a.vdim;
        if (a.mixer_kind == 2) soff += (int64_t)std::max(a.conv - 1, 0) * (nqk + a.heads * a.vdim);
        else soff += (int64_t)a.heads * a.dim + (int64_t)a.heads * (a.vdim + 1);
        mx_big = std::max(mx_big, nqk + 2 * a.heads * a.vdim);
        mx_conv = std::max(mx_conv, a.mixer_kind == 2 ? nqk + a.heads * a.vdim : 0);
      }
      mx_small = std::max(mx_small, (a.mlp_kind == 2 ? a.experts : 0) + (a.mixer_kind >= 2 ? 2 * a.heads : 0));
    }
    if (a.mlp_kind == 1 && a.ff <= 0) return fail(lname(i, "mlp: ff must be positive"));
    if (c.block_kind == 1 && a.mlp_kind == 1) return fail(lname(i, "mlp: the parallel block form has no dense feed-forward"));
    if (c.block_kind == 2 && a.mlp_kind == 2) return fail(lname(i, "mlp: the sandwich block form has no mixture of experts"));
    if (c.block_kind == 3 && a.mlp_kind == 1) return fail(lname(i, "mlp: the pre-norm block form has no dense feed-forward"));
    if (a.mlp_kind == 2) {
      if (a.experts <= 0 || a.top <= 0 || a.expert_ff <= 0 || a.groups <= 0 || a.experts % a.groups || a.keep <= 0 || a.keep > a.groups ||
          a.top > a.keep * (a.experts / a.groups))
        return fail(lname(i, "mlp: inconsistent router (experts, top, groups)"));
    }
    mx_h = std::max(mx_h, a.heads);
    mx_ao = std::max(mx_ao, a.heads * a.vdim);
    if (a.mlp_kind == 1) {
      mx_gu = std::max(mx_gu, 2 * a.ff);
      mx_act = std::max(mx_act, a.ff);
    } else if (a.mlp_kind == 2) {
      mx_gu = std::max(mx_gu, (c.block_kind == 3 ? 2 : 1) * a.shared_ff);
      mx_act = std::max(mx_act, a.shared_ff);
      if (a.expert_act == 2 && (!(a.act_limit > 0.f) || (a.shared_ff > 0 && !(a.shared_limit > 0.f)))) return fail(lname(i, "mlp: limit must be positive"));
      mx_e = std::max(mx_e, a.experts);
      mx_top = std::max(mx_top, a.top);
      mx_hid = std::max(mx_hid, a.top * a.expert_ff);
    }
  }
  page_stride = off;
  slot_stride = soff;
  return true;
}

// upload `src_rows` rows into rows [row0, row0 + src_rows) of a [rows, cols] matrix that is allocated on first use
bool Model::put(Mat& m, int rows, int cols, int row0, const void* src, int src_rows, const std::string& name, int got_rows, int got_cols) {
  if (got_rows != src_rows || got_cols != cols) {
    char b[256];
    snprintf(b, sizeof b, "%s: shape [%d, %d] does not match the [%d, %d] the configuration implies", name.c_str(), got_rows, got_cols, src_rows, cols);
    return fail(b);
  }
  if (!m.d.ptr) {
    m.rows = rows;
    m.cols = cols;
    if (!m.d.alloc_zeros((size_t)rows * cols * es)) return fail("allocation failed for " + name);
  }
  return cu(cudaMemcpy((char*)m.d.ptr + (size_t)row0 * cols * es, src, (size_t)src_rows * cols * es, cudaMemcpyDefault), name.c_str());
}

// the same with destination rows row0, row0 + row_step, ... (interleaving two tensors row by row)
bool Model::put_rows(Mat& m, int rows, int cols, int row0, int row_step, const void* src, int src_rows, const std::string& name, int got_rows, int got_cols) {
  if (got_rows != src_rows || got_cols != cols) {
    char b[256];
    snprintf(b, sizeof b, "%s: shape [%d, %d] does not match the [%d, %d] the configuration implies", name.c_str(), got_rows, got_cols, src_rows, cols);
    return fail(b);
  }
  if (!m.d.ptr) {
    m.rows = rows;
    m.cols = cols;
    if (!m.d.alloc_zeros((size_t)rows * cols * es)) return fail("allocation failed for " + name);
  }
  return cu(cudaMemcpy2D((char*)m.d.ptr + (size_t)row0 * cols * es, (size_t)row_step * cols * es, src, (size_t)cols * es, (size_t)cols * es, src_rows,
                         cudaMemcpyDefault),
            name.c_str());
}

// W_uk [heads * dim, rank] as stored, and a second copy with the contraction axis of the query fold contiguous: [head][rank][dim]
bool Model::put_uk(Layer& L, const void* data, const std::string& name, int rows, int cols) {
  const LayerCfg& a = L.c;
  if (!put(L.uk, a.heads * a.dim, a.kv_rank, 0, data, a.heads * a.dim, name, rows, cols)) return false;
  const size_t n = (size_t)a.heads * a.dim * a.kv_rank;
  std::vector<char> src(n * es), dst(n * es);
  if (!cu(cudaMemcpy(src.data(), data, n * es, cudaMemcpyDefault), name.c_str())) return false;
  for (int h = 0; h < a.heads; ++h)
    for (int d = 0; d < a.dim; ++d)
      for (int r = 0; r < a.kv_rank; ++r)
        memcpy(&dst[(((size_t)h * a.kv_rank + r) * a.dim + d) * es], &src[(((size_t)h * a.dim + d) * a.kv_rank + r) * es], es);
  return put(L.uk_t, a.heads * a.kv_rank, a.dim, 0, dst.data(), a.heads * a.kv_rank, name, a.heads * a.kv_rank, a.dim);
}

// float copy of a small parameter vector that enters fp32 arithmetic only
bool Model::to_f32(const Mat& m, DeviceBuf* out) {
  const long n = (long)m.rows * m.cols;
  if (!m.d.ptr || n <= 0) return fail("parameter vector missing");
  if (!out->alloc_zeros((size_t)n * 4)) return fail("allocation failed");
  return rc(k.pk_convert(m.d.ptr, c.f32, out->ptr, 1, n, st), "parameter conversion");
}

bool Model::load_tensor(const std::string& name, const void* data, int rows, int cols, int is_f32) {
  if ((is_f32 != 0) != (c.f32 != 0)) return fail(name + ": element type differs from the model's");
  const int W = c.width;
  if (name == "embed") return put(embed, c.vocab, W, 0, data, c.vocab, name, rows, cols);
  if (c.block_kind == 2 && name == "embed.norm") return put(embed_norm, 1, W, 0, data, 1, name, rows, cols);
  if (name == "head") return put(head, c.vocab, W, 0, data, c.vocab, name, rows, cols);
  if (name == "final.norm") return put(final_norm, 1, W, 0, data, 1, name, rows, cols);
  if (c.block_kind == 1 && name == "final.norm.b") return put(final_b, 1, W, 0, data, 1, name, rows, cols);
  if (c.block_kind == 1 && name == "final.norm.alpha") return put(final_alpha, 1, 1, 0, data, 1, name, rows, cols);
  if (name.size() < 3 || name[0] != 'l') return fail("unknown tensor " + name);
  const size_t dot = name.find('.');
  if (dot == std::string::npos || dot < 2) return fail("unknown tensor " + name);
  const int li = atoi(name.substr(1, dot - 1).c_str());
  if (li < 0 || li >= c.n_layers) return fail("layer index out of range: " + name);
  Layer& L = layers[li];
  const LayerCfg& a = L.c;
  const std::string sub = name.substr(dot + 1);
  bool ok;
  if (c.block_kind == 1) {
    // parallel block: one Dynamic-Tanh norm; projections stacked [q | k | v (| gate)], few-row fp32 projections [router | za | zb]
    const int H = a.heads, G = a.kv_heads, mk = a.mixer_kind;
    const int nq = (mk == 2 ? G : H) * a.dim, nk = G * a.dim, nv = (mk == 1 ? G : H) * a.vdim, ng = mk == 1 ? 0 : H * a.vdim;
    const int nbig = nq + nk + nv + ng, E0 = a.mlp_kind == 2 ? a.experts : 0, nsmall = E0 + (mk >= 2 ? 2 * H : 0);
    const int taps = a.conv;
    if (sub == "norm1") ok = put(L.norm1, 1, W, 0, data, 1, name, rows, cols);
    else if (sub == "norm1.b") ok = put(L.nb, 1, W, 0, data, 1, name, rows, cols);
    else if (sub == "norm1.alpha") ok = put(L.alpha, 1, 1, 0, data, 1, name, rows, cols);
    else if (sub == "mix.q") ok = put(L.qkv, nbig, W, 0, data, nq, name, rows, cols);
    else if (sub == "mix.k") ok = put(L.qkv, nbig, W, nq, data, nk, name, rows, cols);
    else if (sub == "mix.v") ok = put(L.qkv, nbig, W, nq + nk, data, nv, name, rows, cols);
    else if (mk >= 2 && sub == "mix.g") ok = put(L.qkv, nbig, W, nq + nk + nv, data, ng, name, rows, cols);
    else if (sub == "mix.o") ok = put(L.o, W, H * a.vdim, 0, data, W, name, rows, cols);
    else if (mk == 1 && (sub == "mix.q.b" || sub == "mix.k.b" || sub == "mix.v.b")) {
      const int n = sub[4] == 'q' ? nq : sub[4] == 'k' ? nk : nv, at = sub[4] == 'q' ? 0 : sub[4] == 'k' ? nq : nq + nk;
      if (rows != 1 || cols != n) return fail(name + ": shape does not match the configuration");
      if (!L.qkv_bias.d.ptr) {
        L.qkv_bias.rows = 1;
        L.qkv_bias.cols = nbig;
        if (!L.qkv_bias.d.alloc_zeros((size_t)nbig * es)) return fail("allocation failed for " + name);
      }
      ok = cu(cudaMemcpy((char*)L.qkv_bias.d.ptr + (size_t)at * es, data, (size_t)n * es, cudaMemcpyDefault), name.c_str());
    }
    else if (mk == 1 && sub == "mix.sink") ok = put(L.sink, 1, H, 0, data, 1, name, rows, cols);
    else if (mk == 2 && sub == "mix.q.conv") ok = put(L.conv_w, nq + nk + nv, taps, 0, data, nq, name, rows, cols);
    else if (mk == 2 && sub == "mix.k.conv") ok = put(L.conv_w, nq + nk + nv, taps, nq, data, nk, name, rows, cols);
    else if (mk == 2 && sub == "mix.v.conv") ok = put(L.conv_w, nq + nk + nv, taps, nq + nk, data, nv, name, rows, cols);
    else if (mk == 2 && sub == "mix.a") ok = put(L.small, nsmall, W, E0, data, H, name, rows, cols);
    else if (mk == 2 && sub == "mix.b") ok = put(L.small, nsmall, W, E0 + H, data, H, name, rows, cols);
    else if (mk == 3 && sub == "mix.f") ok = put(L.small, nsmall, W, E0, data, H, name, rows, cols);
    else if (mk == 3 && sub == "mix.i") ok = put(L.small, nsmall, W, E0 + H, data, H, name, rows, cols);
    else if (mk == 2 && sub == "mix.A_log") ok = put(L.p0, 1, H, 0, data, 1, name, rows, cols);
    else if (mk == 2 && sub == "mix.dt_bias") ok = put(L.p1, 1, H, 0, data, 1, name, rows, cols);
    else if (mk == 3 && sub == "mix.i.b") ok = put(L.p0, 1, H, 0, data, 1, name, rows, cols);
    else if (mk == 3 && sub == "mix.f.b") ok = put(L.p1, 1, H, 0, data, 1, name, rows, cols);
    else if (mk == 2 && sub == "mix.norm") ok = put(L.hnorm, 1, a.vdim, 0, data, 1, name, rows, cols);
    else if (mk == 3 && sub == "mix.norm") ok = put(L.hnorm, 1, H * a.vdim, 0, data, 1, name, rows, cols);
    else if (a.mlp_kind == 2 && sub == "mlp.router") ok = put(L.small, nsmall, W, 0, data, a.experts, name, rows, cols);
    else if (a.mlp_kind == 2 && sub == "mlp.correction") ok = put(L.corr, 1, a.experts, 0, data, 1, name, rows, cols);
    else if (a.mlp_kind == 2 && sub.rfind("mlp.e", 0) == 0) {
      const size_t d2 = sub.find('.', 5);
      if (d2 == std::string::npos) return fail("unknown tensor " + name);
      const int e = atoi(sub.substr(5, d2 - 5).c_str());
      const std::string part = sub.substr(d2 + 1);
      if (e < 0 || e >= a.experts) return fail("expert index out of range: " + name);
      const int ff = a.expert_ff;
      if (a.expert_act == 1 && part == "gate") ok = put_rows(L.e_up, a.experts * 2 * ff, W, e * 2 * ff, 2, data, ff, name, rows, cols);
      else if (a.expert_act == 1 && part == "up") ok = put_rows(L.e_up, a.experts * 2 * ff, W, e * 2 * ff + 1, 2, data, ff, name, rows, cols);
      else if (a.expert_act == 0 && part == "up") ok = put(L.e_up, a.experts * ff, W, e * ff, data, ff, name, rows, cols);
      else if (part == "down") ok = put(L.e_down, a.experts * W, ff, e * W, data, W, name, rows, cols);
      else return fail("unknown tensor " + name);
    } else {
      return fail("unknown tensor " + name + " for the configuration of layer " + std::to_string(li));
    }
    if (ok) L.got.insert(sub);
    return ok;
  }
  if (c.block_kind == 2) {
    // sandwich block: [q | k | v (| g) (| rg1)] (attention) or [q | dkv (| rg1)] (latent attention) stacked into one projection
    const int H = a.heads, G = a.kv_heads, mk = a.mixer_kind, rg = c.gated_residual ? W : 0;
    const int nq = mk == 1 ? H * a.dim : H * (a.dim + a.rot_dim), nk = mk == 1 ? G * a.dim : a.kv_rank + a.rot_dim, nv = mk == 1 ? G * a.vdim : 0;
    const int ng = mk == 1 && a.out_gate ? H * a.vdim : 0, nbig = nq + nk + nv + ng + rg;
    auto vec = [&](Mat& m, int n, int total, int at) {  // a vector stored as a slice of a [1, total] row
      if (rows != 1 || cols != n) return fail(name + ": shape does not match the configuration");
      if (!m.d.ptr) {
        m.rows = 1;
        m.cols = total;
        if (!m.d.alloc_zeros((size_t)total * es)) return fail("allocation failed for " + name);
      }
      return cu(cudaMemcpy((char*)m.d.ptr + (size_t)at * es, data, (size_t)n * es, cudaMemcpyDefault), name.c_str());
    };
    if (sub == "norm1") ok = put(L.norm1, 1, W, 0, data, 1, name, rows, cols);
    else if (sub == "norm1b") ok = put(L.norm1b, 1, W, 0, data, 1, name, rows, cols);
    else if (a.mlp_kind && sub == "norm2") ok = put(L.norm2, 1, W, 0, data, 1, name, rows, cols);
    else if (a.mlp_kind && sub == "norm2b") ok = put(L.norm2b, 1, W, 0, data, 1, name, rows, cols);
    else if (sub == "mix.q") ok = put(L.qkv, nbig, W, 0, data, nq, name, rows, cols);
    else if (mk == 1 && sub == "mix.k") ok = put(L.qkv, nbig, W, nq, data, nk, name, rows, cols);
    else if (mk == 1 && sub == "mix.v") ok = put(L.qkv, nbig, W, nq + nk, data, nv, name, rows, cols);
    else if (ng && sub == "mix.g") ok = put(L.qkv, nbig, W, nq + nk + nv, data, ng, name, rows, cols);
    else if (rg && sub == "rg1") ok = put(L.qkv, nbig, W, nq + nk + nv + ng, data, W, name, rows, cols);
    else if (rg && sub == "rg1.b") ok = put(L.rg1_bias, 1, W, 0, data, 1, name, rows, cols);
    else if (rg && a.mlp_kind && sub == "rg2") ok = put(L.rg2, W, W, 0, data, W, name, rows, cols);
    else if (rg && a.mlp_kind && sub == "rg2.b") ok = put(L.rg2_bias, 1, W, 0, data, 1, name, rows, cols);
    else if (mk == 1 && a.proj_bias && sub == "mix.q.b") ok = vec(L.qkv_bias, nq, nq + nk + nv, 0);
    else if (mk == 1 && a.proj_bias && sub == "mix.k.b") ok = vec(L.qkv_bias, nk, nq + nk + nv, nq);
    else if (mk == 1 && a.proj_bias && sub == "mix.v.b") ok = vec(L.qkv_bias, nv, nq + nk + nv, nq + nk);
    else if (mk == 1 && a.proj_bias && sub == "mix.o.b") ok = put(L.o_bias, 1, W, 0, data, 1, name, rows, cols);
    else if (mk == 1 && a.sink_kind == 0 && sub == "mix.sink") ok = put(L.sink, 1, H, 0, data, 1, name, rows, cols);
    else if (mk == 0 && sub == "mix.dkv") ok = put(L.qkv, nbig, W, nq, data, nk, name, rows, cols);
    else if (mk == 0 && sub == "mix.dkv.norm") ok = put(L.dkv_norm, 1, a.kv_rank, 0, data, 1, name, rows, cols);
    else if (mk == 0 && sub == "mix.uk") ok = put_uk(L, data, name, rows, cols);
    else if (mk == 0 && sub == "mix.uv") ok = put(L.uv, H * a.vdim, a.kv_rank, 0, data, H * a.vdim, name, rows, cols);
    else if (mk == 0 && a.sink_kind == 0 && sub == "mix.sink") ok = put(L.sink, 1, H, 0, data, 1, name, rows, cols);
    else if (sub == "mix.o") ok = put(L.o, W, H * a.vdim, 0, data, W, name, rows, cols);
    else if (a.mlp_kind == 1 && sub == "mlp.gate") ok = put(L.gate_up, 2 * a.ff, W, 0, data, a.ff, name, rows, cols);
    else if (a.mlp_kind == 1 && sub == "mlp.up") ok = put(L.gate_up, 2 * a.ff, W, a.ff, data, a.ff, name, rows, cols);
    else if (a.mlp_kind == 1 && sub == "mlp.down") ok = put(L.down, W, a.ff, 0, data, W, name, rows, cols);
    else return fail("unknown tensor " + name + " for the configuration of layer " + std::to_string(li));
    if (ok) L.got.insert(sub);
    return ok;
  }
  if (c.block_kind == 3) {
    // pre-norm block: [q | k | v] (attention) or [q | k | in] (attention beside a state-space branch) stacked into one projection;
    // expert gate / up rows interleaved; the shared expert's [gate ; up] stacked
    if (L.wsrc != li) return fail(name + ": layer " + std::to_string(li) + " runs with the weights of layer " + std::to_string(L.wsrc));
    const int H = a.heads, G = a.kv_heads, mk = a.mixer_kind;
    const int nq = H * a.dim, nk = G * a.dim, nv = mk == 1 && !a.values_are_keys ? G * a.vdim : 0;
    const int inner = mk == 4 ? a.ssm_heads * a.ssm_vdim : 0, C = mk == 4 ? inner + 2 * a.ssm_groups * a.ssm_state : 0;
    const int nin = mk == 4 ? inner + C + a.ssm_heads : 0, nbig = nq + nk + nv + nin;
    const std::string am = mk == 4 ? "mix.left." : "mix.";  // where the attention's tensors live
    const int nw = a.qk_norm == 2 ? 0 : a.dim;             // norm weight per head (shared) or over the whole projection
    if (sub == "norm1") ok = put(L.norm1, 1, W, 0, data, 1, name, rows, cols);
    else if (a.mlp_kind && sub == "norm2") ok = put(L.norm2, 1, W, 0, data, 1, name, rows, cols);
    else if (sub == am + "q") ok = put(L.qkv, nbig, W, 0, data, nq, name, rows, cols);
    else if (sub == am + "k") ok = put(L.qkv, nbig, W, nq, data, nk, name, rows, cols);
    else if (nv && sub == am + "v") ok = put(L.qkv, nbig, W, nq + nk, data, nv, name, rows, cols);
    else if (a.qk_norm && sub == am + "q.norm") ok = put(L.qn, 1, nw ? nw : nq, 0, data, 1, name, rows, cols);
    else if (a.qk_norm && sub == am + "k.norm") ok = put(L.kn, 1, nw ? nw : nk, 0, data, 1, name, rows, cols);
    else if (a.sink_kind == 0 && sub == am + "sink") ok = put(L.sink, 1, H, 0, data, 1, name, rows, cols);
    else if (sub == am + "o") ok = put(L.o, W, H * a.vdim, 0, data, W, name, rows, cols);
    else if (mk == 4 && sub == "mix.right.in") ok = put(L.qkv, nbig, W, nq + nk, data, nin, name, rows, cols);
    else if (mk == 4 && sub == "mix.right.conv") ok = put(L.conv_w, C, a.conv, 0, data, C, name, rows, cols);
    else if (mk == 4 && sub == "mix.right.conv.b") ok = put(L.conv_b, 1, C, 0, data, 1, name, rows, cols);
    else if (mk == 4 && sub == "mix.right.A_log") ok = put(L.p0, 1, a.ssm_heads, 0, data, 1, name, rows, cols);
    else if (mk == 4 && sub == "mix.right.dt_bias") ok = put(L.p1, 1, a.ssm_heads, 0, data, 1, name, rows, cols);
    else if (mk == 4 && sub == "mix.right.D") ok = put(L.p2, 1, a.ssm_heads, 0, data, 1, name, rows, cols);
    else if (mk == 4 && sub == "mix.right.norm") ok = put(L.hnorm, 1, inner, 0, data, 1, name, rows, cols);
    else if (mk == 4 && sub == "mix.right.o") ok = put(L.o2, W, inner, 0, data, W, name, rows, cols);
    else if (mk == 4 && sub == "mix.left.out") ok = put(L.lout, 1, W, 0, data, 1, name, rows, cols);
    else if (mk == 4 && sub == "mix.right.out") ok = put(L.rout, 1, W, 0, data, 1, name, rows, cols);
    else if (a.mlp_kind == 2 && sub == "mlp.router") ok = put(L.router, a.experts, W, 0, data, a.experts, name, rows, cols);
    else if (a.mlp_kind == 2 && sub == "mlp.router.b") ok = put(L.corr, 1, a.experts, 0, data, 1, name, rows, cols);
    else if (a.mlp_kind == 2 && a.shared_ff > 0 && sub == "mlp.shared.gate") ok = put(L.gate_up, 2 * a.shared_ff, W, 0, data, a.shared_ff, name, rows, cols);
    else if (a.mlp_kind == 2 && a.shared_ff > 0 && sub == "mlp.shared.up") ok = put(L.gate_up, 2 * a.shared_ff, W, a.shared_ff, data, a.shared_ff, name, rows, cols);
    else if (a.mlp_kind == 2 && a.shared_ff > 0 && sub == "mlp.shared.down") ok = put(L.s_down, W, a.shared_ff, 0, data, W, name, rows, cols);
    else if (a.mlp_kind == 2 && sub.rfind("mlp.e", 0) == 0) {
      const size_t d2 = sub.find('.', 5);
      if (d2 == std::string::npos) return fail("unknown tensor " + name);
      const int e = atoi(sub.substr(5, d2 - 5).c_str());
      const std::string part = sub.substr(d2 + 1);
      if (e < 0 || e >= a.experts) return fail("expert index out of range: " + name);
      const int ff = a.expert_ff;
      if (part == "gate") ok = put_rows(L.e_up, a.experts * 2 * ff, W, e * 2 * ff, 2, data, ff, name, rows, cols);
      else if (part == "up") ok = put_rows(L.e_up, a.experts * 2 * ff, W, e * 2 * ff + 1, 2, data, ff, name, rows, cols);
      else if (part == "down") ok = put(L.e_down, a.experts * W, ff, e * W, data, W, name, rows, cols);
      else return fail("unknown tensor " + name);
    } else {
      return fail("unknown tensor " + name + " for the configuration of layer " + std::to_string(li));
    }
    if (ok) L.got.insert(sub);
    return ok;
  }
  if (sub == "norm1") ok = put(L.norm1, 1, W, 0, data, 1, name, rows, cols);
  else if (sub == "norm2") ok = put(L.norm2, 1, W, 0, data, 1, name, rows, cols);
  else if (sub == "mix.q") ok = put(L.q, a.heads * (a.dim + a.rot_dim), W, 0, data, a.heads * (a.dim + a.rot_dim), name, rows, cols);
  else if (sub == "mix.dkv" && a.kv_from < 0) ok = put(L.dkv, a.kv_rank + a.rot_dim, W, 0, data, a.kv_rank + a.rot_dim, name, rows, cols);
  else if (sub == "mix.dkv.norm" && a.kv_from < 0) ok = put(L.dkv_norm, 1, a.kv_rank, 0, data, 1, name, rows, cols);
  else if (sub == "mix.uk") ok = put_uk(L, data, name, rows, cols);
  else if (sub == "mix.uv") ok = put(L.uv, a.heads * a.vdim, a.kv_rank, 0, data, a.heads * a.vdim, name, rows, cols);
  else if (sub == "mix.sink") ok = put(L.sink, 1, a.heads, 0, data, 1, name, rows, cols);
  else if (sub == "mix.g") ok = put(L.g, a.heads, W, 0, data, a.heads, name, rows, cols);
  else if (sub == "mix.o") ok = put(L.o, W, a.heads * a.vdim, 0, data, W, name, rows, cols);
  else if (a.mlp_kind == 1 && sub == "mlp.gate") ok = put(L.gate_up, 2 * a.ff, W, 0, data, a.ff, name, rows, cols);
  else if (a.mlp_kind == 1 && sub == "mlp.up") ok = put(L.gate_up, 2 * a.ff, W, a.ff, data, a.ff, name, rows, cols);
  else if (a.mlp_kind == 1 && sub == "mlp.down") ok = put(L.down, W, a.ff, 0, data, W, name, rows, cols);
  else if (a.mlp_kind == 2 && sub == "mlp.router") ok = put(L.router, a.experts, W, 0, data, a.experts, name, rows, cols);
  else if (a.mlp_kind == 2 && a.shared_ff > 0 && sub == "mlp.shared.up") ok = put(L.s_up, a.shared_ff, W, 0, data, a.shared_ff, name, rows, cols);
  else if (a.mlp_kind == 2 && a.shared_ff > 0 && sub == "mlp.shared.down") ok = put(L.s_down, W, a.shared_ff, 0, data, W, name, rows, cols);
  else if (a.mlp_kind == 2 && a.shared_ff > 0 && sub == "mlp.shared.sg") ok = put(L.s_gate, 1, W, 0, data, 1, name, rows, cols);
  else if (a.mlp_kind == 2 && sub.rfind("mlp.e", 0) == 0) {
    const size_t d2 = sub.find('.', 5);
    if (d2 == std::string::npos) return fail("unknown tensor " + name);
    const int e = atoi(sub.substr(5, d2 - 5).c_str());
    const std::string part = sub.substr(d2 + 1);
    if (e < 0 || e >= a.experts) return fail("expert index out of range: " + name);
    if (part == "up") ok = put(L.e_up, a.experts * a.expert_ff, W, e * a.expert_ff, data, a.expert_ff, name, rows, cols);
    else if (part == "down") ok = put(L.e_down, a.experts * W, a.expert_ff, e * W, data, W, name, rows, cols);
    else return fail("unknown tensor " + name);
  } else {
    return fail("unknown tensor " + name + " for the configuration of layer " + std::to_string(li));
  }
  if (ok) L.got.insert(sub);
  return ok;
}

// angular frequency of every rotated pair; with YaRN scaling, pairs that turn fewer than `slow` times over the original
// context are slowed by `factor`, pairs that turn more than `fast` times are kept, a linear ramp over the pair index blends
// Scaling by wavelength (scaling_kind 1): a pair whose wavelength 2 pi / w is below original / high keeps w, one above original / low
// turns at w / factor, and between the two the blend is linear in original / wavelength.
static void rotary_table(const LayerCfg& a, std::vector<float>* f, float* mag) {
  const int half = a.rot_dims / 2;
  f->resize(std::max(half, 1));
  *mag = 1.f;
  if (a.has_scaling && a.scaling_kind == 1) {
    const double factor = a.s_factor, orig = a.s_original, high = a.s_fast, low = a.s_slow;
    for (int i = 0; i < half; ++i) {
      const double w = std::pow((double)a.rot_base, -2.0 * i / a.rot_dims), wavelength = 2.0 * M_PI / w;
      double r = w;
      if (wavelength > orig / low) r = w / factor;
      else if (!(wavelength < orig / high)) {
        const double blend = (orig / wavelength - low) / (high - low);
        r = (1.0 - blend) * w / factor + blend * w;
      }
      (*f)[i] = (float)r;
    }
    return;
  }
  double lo = 0, hi = 0;
  if (a.has_scaling) {
    auto pair_of = [&](double turns) { return a.rot_dims * std::log((double)a.s_original / (2.0 * M_PI * turns)) / (2.0 * std::log((double)a.rot_base)); };
    lo = std::max(std::floor(pair_of(a.s_fast)), 0.0);
    hi = std::min(std::ceil(pair_of(a.s_slow)), (double)a.rot_dims - 1.0);
    *mag = (float)(0.1 * std::log((double)a.s_factor) + 1.0);
  }
  for (int i = 0; i < half; ++i) {
    double w = std::pow((double)a.rot_base, -2.0 * i / a.rot_dims);
    if (a.has_scaling) {
      const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
      w = w / a.s_factor * ramp + w * (1.0 - ramp);
    }
    (*f)[i] = (float)w;
  }
}

bool Model::finalize() {
  if (!embed.d.ptr || !head.d.ptr || !final_norm.d.ptr) return fail("embed / head / final.norm missing");
  if (c.block_kind == 2 && !embed_norm.d.ptr) return fail("embed.norm missing");
  if (c.block_kind == 2 && !zero_sink.alloc_zeros((size_t)std::max(mx_h, 1) * es)) return fail("allocation failed");
  if (c.block_kind == 1 && (!final_b.d.ptr || !final_alpha.d.ptr || !to_f32(final_alpha, &final_alpha32))) return fail("final.norm.b / final.norm.alpha missing");
  if (slot_stride > 0 && !state.alloc_zeros((size_t)c.max_requests * slot_stride * 4)) return fail("state slot allocation failed");
  if (page_stride == 0) page_stride = 8;  // no layer keeps a paged cache: the pool only counts tokens
  for (int i = 0; i < c.n_layers; ++i) {
    Layer& L = layers[i];
    const LayerCfg& a = L.c;
    std::vector<std::string> need;
    if (c.block_kind == 3) {
      if (L.wsrc == i) {
        const std::string am = a.mixer_kind == 4 ? "mix.left." : "mix.";
        need = {"norm1", am + "q", am + "k", am + "o"};
        if (a.mixer_kind == 1 && !a.values_are_keys) need.push_back(am + "v");
        if (a.qk_norm) need.insert(need.end(), {am + "q.norm", am + "k.norm"});
        if (a.sink_kind == 0) need.push_back(am + "sink");
        if (a.mixer_kind == 4)
          for (const char* n : {"in", "conv", "conv.b", "A_log", "dt_bias", "D", "norm", "o", "out"}) need.push_back(std::string("mix.right.") + n);
        if (a.mixer_kind == 4) need.push_back("mix.left.out");
        if (a.mlp_kind) need.insert(need.end(), {"norm2", "mlp.router.b"});
      }
    } else if (c.block_kind == 0) {
      need = {"norm1", "mix.q", "mix.uk", "mix.uv", "mix.sink", "mix.g", "mix.o"};
      if (a.kv_from < 0) need.insert(need.end(), {"mix.dkv", "mix.dkv.norm"});
      if (a.mlp_kind) need.push_back("norm2");
    } else if (c.block_kind == 2) {
      need = {"norm1", "norm1b", "mix.q", "mix.o"};
      if (a.mixer_kind == 1) need.insert(need.end(), {"mix.k", "mix.v"});
      else need.insert(need.end(), {"mix.dkv", "mix.dkv.norm", "mix.uk", "mix.uv"});
      if (a.mixer_kind == 1 && a.proj_bias) need.insert(need.end(), {"mix.q.b", "mix.k.b", "mix.v.b", "mix.o.b"});
      if (a.mixer_kind == 1 && a.out_gate) need.push_back("mix.g");
      if (a.sink_kind == 0) need.push_back("mix.sink");
      if (c.gated_residual) need.insert(need.end(), {"rg1", "rg1.b"});
      if (a.mlp_kind) need.insert(need.end(), {"norm2", "norm2b"});
      if (a.mlp_kind && c.gated_residual) need.insert(need.end(), {"rg2", "rg2.b"});
    } else {
      need = {"norm1", "norm1.b", "norm1.alpha", "mix.q", "mix.k", "mix.v", "mix.o"};
      if (a.mixer_kind == 1) need.insert(need.end(), {"mix.q.b", "mix.k.b", "mix.v.b", "mix.sink"});
      if (a.mixer_kind == 2) need.insert(need.end(), {"mix.q.conv", "mix.k.conv", "mix.v.conv", "mix.a", "mix.b", "mix.A_log", "mix.dt_bias", "mix.norm", "mix.g"});
      if (a.mixer_kind == 3) need.insert(need.end(), {"mix.i", "mix.f", "mix.i.b", "mix.f.b", "mix.norm", "mix.g"});
      if (a.mlp_kind == 2) need.push_back("mlp.correction");
    }
    if (a.mlp_kind == 1) need.insert(need.end(), {"mlp.gate", "mlp.up", "mlp.down"});
    if (a.mlp_kind == 2 && L.wsrc == i) {
      need.push_back("mlp.router");
      for (int e = 0; e < a.experts; ++e) {
        if (a.expert_act >= 1) need.push_back("mlp.e" + std::to_string(e) + ".gate");
        need.push_back("mlp.e" + std::to_string(e) + ".up");
        need.push_back("mlp.e" + std::to_string(e) + ".down");
      }
      if (a.shared_ff > 0) need.insert(need.end(), {"mlp.shared.up", "mlp.shared.down", c.block_kind == 3 ? "mlp.shared.gate" : "mlp.shared.sg"});
    }
    for (auto& n : need)
      if (!L.got.count(n)) return fail("tensor " + lname(i, n.c_str()) + " is missing");
    if (c.block_kind == 1) {
      if (!to_f32(L.alpha, &L.alpha32)) return false;
      if (a.mlp_kind == 2 && !to_f32(L.corr, &L.corr32)) return false;
      if (a.mixer_kind >= 2 && (!to_f32(L.p0, &L.p0_32) || !to_f32(L.p1, &L.p1_32))) return false;
      if (a.mixer_kind != 1) continue;  // only attention rotates
    }
    if (c.block_kind == 3 && L.wsrc == i) {
      if (a.mlp_kind == 2 && !to_f32(L.corr, &L.corr32)) return false;
      if (a.mixer_kind == 4 && (!to_f32(L.p0, &L.p0_32) || !to_f32(L.p1, &L.p1_32) || !to_f32(L.p2, &L.p2_32))) return false;
    }
    if (c.block_kind >= 2 && a.rot_dims == 0) continue;  // nothing rotates
    std::vector<float> f;
    rotary_table(a, &f, &L.mag);
    if (!L.freq.alloc_zeros(f.size() * 4) || !cu(cudaMemcpy(L.freq.ptr, f.data(), f.size() * 4, cudaMemcpyHostToDevice), "rotary table"))
      return fail("rotary table upload failed");
  }
  if (c.num_pages <= 0) {  // a share of what is free, as the other hosts size their pools
    size_t fr = 0, tot = 0;
    cudaMemGetInfo(&fr, &tot);
    c.num_pages = (int)std::min<size_t>((size_t)(fr * 0.85) / ((size_t)page_stride * es), (size_t)1 << 20);
  }
  c.num_pages += 1;  // page 0 is never handed out (padding rows of captured steps point there)
  if (!cache.alloc_zeros((size_t)c.num_pages * page_stride * es)) return fail("cache pool allocation failed");
  pool.init(c.num_pages);
  std::vector<int> pad;
  pool.acquire(1, &pad);
  reqs.assign(c.max_requests, pq::KvState());
  fresh.assign(c.max_requests, 0);
  if (cudaMallocHost((void**)&sampled_h, 4096) != cudaSuccess) return fail("pinned allocation failed");
  if (!top1_val.alloc_zeros(64) || !top1_states.alloc_zeros(1 << 16)) return fail("sampler scratch allocation failed");
  finalized = true;
  return cu(cudaStreamSynchronize(st), "finalize");
}

bool Model::ensure_scratch(int T, int R) {
  bool ok = true;
  if (T > cap_t) {
    cudaStreamSynchronize(st);
    drop_graphs();
    const size_t n = ((size_t)T + 63) / 64 * 64, W = c.width;
    ok = x.alloc_uninit(n * W * 4) && xa.alloc_uninit(n * W * es) && q.alloc_uninit(n * mx_q * es) && dkv.alloc_uninit(n * mx_dkv * es) &&
         qa.alloc_uninit(n * mx_qa * es) && gate.alloc_uninit(n * mx_h * 4) && olat.alloc_uninit(n * mx_olat * es) &&
         ao.alloc_uninit(n * mx_ao * es) && mix.alloc_uninit(n * W * es) && gu.alloc_uninit(n * std::max(mx_gu, 1) * es) &&
         act.alloc_uninit(n * std::max(mx_act, 1) * es) && z.alloc_uninit(n * std::max(mx_e, 1) * 4) && ids.alloc_uninit(n * std::max(mx_top, 1) * 4) &&
         wts.alloc_uninit(n * std::max(mx_top, 1) * 4) && hid.alloc_uninit(n * std::max(mx_hid, 1) * es) && yf.alloc_uninit(n * W * 4) &&
         sgl.alloc_uninit(n * 4) && sh.alloc_uninit(n * W * es);
    if (ok && c.block_kind == 1)
      ok = h32.alloc_uninit(n * W * 4) && big.alloc_uninit(n * std::max(mx_big, 1) * es) && convo.alloc_uninit(n * std::max(mx_conv, 1) * es) &&
           zs.alloc_uninit(n * std::max(mx_small, 1) * 4) && orec.alloc_uninit(n * std::max(mx_ao, 1) * 4) && den.alloc_uninit(n * std::max(mx_h, 1) * 4);
    if (ok && c.block_kind == 2) ok = big.alloc_uninit(n * std::max(mx_big, 1) * es) && rgbuf.alloc_uninit(n * W * es);
    if (ok && c.block_kind == 3)
      ok = h32.alloc_uninit(n * W * 4) && big.alloc_uninit(n * std::max(mx_big, 1) * es) && convo.alloc_uninit(n * std::max(mx_conv, 1) * es) &&
           orec.alloc_uninit(n * std::max(mx_inner, 1) * 4) && ao2.alloc_uninit(n * std::max(mx_inner, 1) * es) && mix2.alloc_uninit(n * W * es);
    if (ok && !c.f32 && (int)n >= kGroupedMinTokens) {  // bucketed experts for prompt portions
      long ws = 0;
      for (auto& L : layers)
        if (L.c.mlp_kind == 2) ws = std::max(ws, k.pk_moe_grouped_workspace_bytes((int)n, L.c.top, L.c.experts, c.width, L.c.expert_ff));
      ok = ws == 0 || moe_ws.alloc_uninit((size_t)ws);
    }
    if (ok) cap_t = (int)n;
  }
  if (ok && R > cap_r) {
    cudaStreamSynchronize(st);
    drop_graphs();
    const size_t n = ((size_t)R + 15) / 16 * 16;
    ok = xr.alloc_uninit(n * c.width * es) && logits_e.alloc_uninit(n * c.vocab * es) && logits_f.alloc_uninit(n * c.vocab * 4) &&
         logits_bf.alloc_uninit(n * c.vocab * 2) && sampled_d.alloc_zeros(n * 4);
    if (ok) cap_r = (int)n;
  }
  return ok ? true : fail("scratch allocation failed");
}

// Y[N, W.rows] = X[N, W.cols] W^T: the library's tensor-core GEMM / streaming GEMV in bf16, plain FMA in fp32
bool Model::lin(const Mat& W, const void* X, void* Y, int N) {
  if (c.f32)
    return rc(k.pk_gemm_strided(X, W.d.ptr, Y, nullptr, N, W.rows, W.cols, W.cols, 1, W.cols, W.rows, 1, 0, 0, 0, 0, 0, 1, st), "linear layer");
  k.gemm_cuda((const pk_bf16*)W.d.ptr, (const pk_bf16*)X, (pk_bf16*)Y, W.rows, N, W.cols, st);
  return true;
}

// out[T, W.rows] (fp32) = residual W^T for the few-row projections (gates, router): from the fp32 residual per token, or -- for
// a prompt portion in bf16 -- from its bf16 copy on the tensor cores (fp32 accumulation and output either way)
bool Model::skinny(const Mat& W, float* out, int T, const char* what, const float* in32) {
  if (!in32) in32 = (const float*)x.ptr;
  if (!c.f32 && T >= kGroupedMinTokens) {
    const int r = k.pk_proj_rows_f32out(W.d.ptr, xa.ptr, out, W.rows, W.cols, T, st);
    if (r != -2) return rc(r, what);
  }
  return rc(k.pk_res32_skinny_proj(W.d.ptr, in32, out, W.rows, W.cols, T, c.f32, st), what);
}

bool Model::run_layer(int li, int T, int max_kv, const int* d_pos, const int* d_req, const int* d_poff, const int* d_pages) {
  Layer& L = layers[li];
  const LayerCfg& a = L.c;
  const int W = c.width, f32 = c.f32, H = a.heads, r = a.kv_rank, rd = a.rot_dim, D = r + rd;
  char* pool_base = (char*)cache.ptr + (size_t)L.cache_off * es;
  // ---- mixer
  if (!lin(L.q, xa.ptr, q.ptr, T)) return false;
  if (a.kv_from < 0) {
    if (!lin(L.dkv, xa.ptr, dkv.ptr, T)) return false;
    if (!rc(k.pk_latent_kv_append(dkv.ptr, L.dkv_norm.d.ptr, d_pos, d_req, d_poff, d_pages, pool_base, page_stride, c.page_size, r, rd, a.rot_dims,
                                  (const float*)L.freq.ptr, L.mag, c.eps, T, f32, st),
            "latent cache append"))
      return false;
  }
  // fold the unrotated query onto the latent (per head: qa[:, :r] = q_unrotated W_uk[h]), rotate the other part beside it
  if (!rc(k.pk_gemm_strided(q.ptr, L.uk_t.d.ptr, qa.ptr, nullptr, T, r, a.dim, (long)H * (a.dim + rd), 1, a.dim, (long)H * D, H, a.dim + rd,
                            (long)a.dim * r, D, 0, 0, f32, st),
          "query fold"))
    return false;
  if (rd > 0 && !rc(k.pk_rope_slice(q.ptr, qa.ptr, d_pos, (const float*)L.freq.ptr, L.mag, T, H, a.dim + rd, a.dim, D, r, rd, a.rot_dims, f32, st),
                    "query rotation"))
    return false;
  if (!skinny(L.g, (float*)gate.ptr, T, "output gate")) return false;
  if (!rc(k.pk_latent_attention(qa.ptr, pool_base, L.sink.d.ptr, d_pos, d_req, d_poff, d_pages, olat.ptr, page_stride, c.page_size, T, H, r, rd,
                                a.scale, max_kv, f32, st),
          "latent attention"))
    return false;
  // values: ao[:, h] = logistic(gate[:, h]) * (o_lat[:, h] W_uv[h]^T)
  if (!rc(k.pk_gemm_strided(olat.ptr, L.uv.d.ptr, ao.ptr, (const float*)gate.ptr, T, a.vdim, r, (long)H * r, 1, r, (long)H * a.vdim, H, r,
                            (long)a.vdim * r, a.vdim, H, 2, f32, st),
          "value expansion"))
    return false;
  if (!lin(L.o, ao.ptr, mix.ptr, T)) return false;
  if (!rc(k.pk_res32_offset_norm_add(mix.ptr, f32, L.norm1.d.ptr, (float*)x.ptr, xa.ptr, W, T, c.eps, f32, st), "norm1")) return false;
  // ---- feed-forward
  if (a.mlp_kind == 1) {
    // bf16: gate | up projection with the SwiGLU activation in its epilogue (the library's fused GEMV for <= 4 tokens, its
    // tensor-core GEMM above; the same rounding points as the two launches they replace, which remain the fallback)
    bool fused = false;
    if (!f32 && T <= 4) {
      pk_b200_gemv_args g{};
      g.W = (const pk_bf16*)L.gate_up.d.ptr;
      g.X = (const pk_bf16*)xa.ptr;
      g.Y[0] = (pk_bf16*)act.ptr;
      g.seg_rows[0] = a.ff;
      g.M = a.ff;
      g.N = T;
      g.K = W;
      g.epi = 1;
      fused = k.pk_b200_gemv_fused(&g, st) == 0;
    } else if (!f32) {
      fused = k.pk_b200_gemm_swiglu((const pk_bf16*)L.gate_up.d.ptr, (const pk_bf16*)xa.ptr, (pk_bf16*)act.ptr, a.ff, T, W, st) == 0;
    }
    if (!fused) {
      if (!lin(L.gate_up, xa.ptr, gu.ptr, T)) return false;
      if (!rc(k.pk_act(gu.ptr, act.ptr, a.ff, T, 0, f32, st), "SwiGLU")) return false;
    }
    if (!lin(L.down, act.ptr, mix.ptr, T)) return false;
    if (!rc(k.pk_res32_offset_norm_add(mix.ptr, f32, L.norm2.d.ptr, (float*)x.ptr, xa.ptr, W, T, c.eps, f32, st), "norm2")) return false;
  } else if (a.mlp_kind == 2) {
    if (!skinny(L.router, (float*)z.ptr, T, "router")) return false;
    if (!rc(k.pk_router_grouped_topk((const float*)z.ptr, (int*)ids.ptr, (float*)wts.ptr, T, a.experts, a.top, a.groups, a.keep, a.route_scale, st),
            "router top-k"))
      return false;
    const void* shared = nullptr;
    if (a.shared_ff > 0) {
      if (!lin(L.s_up, xa.ptr, gu.ptr, T)) return false;
      if (!rc(k.pk_act(gu.ptr, act.ptr, a.shared_ff, T, 1, f32, st), "shared expert activation")) return false;
      if (!lin(L.s_down, act.ptr, sh.ptr, T)) return false;
      if (!skinny(L.s_gate, (float*)sgl.ptr, T, "shared expert gate")) return false;
      shared = sh.ptr;
    }
    if (!run_experts(L, T, shared, (const float*)sgl.ptr)) return false;
    if (!rc(k.pk_res32_offset_norm_add(yf.ptr, 1, L.norm2.d.ptr, (float*)x.ptr, xa.ptr, W, T, c.eps, f32, st), "norm2")) return false;
  }
  if (keep_trail)
    return cu(cudaMemcpyAsync((char*)trail.ptr + (size_t)li * T * W * 4, x.ptr, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, st), "trail copy");
  return true;
}

// routed experts of one layer for the tokens in xa: router logits are in zs (block 1) or z (block 0); result in yf (fp32)
bool Model::run_experts(const Layer& L, int T, const void* shared, const float* shared_gate) {
  const LayerCfg& a = L.c;
  const int W = c.width, f32 = c.f32;
  // many tokens: rows bucketed by expert on the tensor cores; a few tokens: per token, reading only the chosen experts' weights
  int grouped = -2;
  if (!f32 && T >= kGroupedMinTokens && moe_ws.ptr) {
    grouped = k.pk_moe_grouped_act_p(xa.ptr, L.e_up.d.ptr, L.e_down.d.ptr, (const int*)ids.ptr, (const float*)wts.ptr, shared, shared_gate,
                                     (float*)yf.ptr, moe_ws.ptr, T, a.top, a.experts, W, a.expert_ff, a.expert_act, a.act_limit, a.act_slope, st);
    if (grouped != -2 && !rc(grouped, "experts (grouped)")) return false;
  }
  if (grouped == -2 && !rc(k.pk_moe_up_act_p(xa.ptr, L.e_up.d.ptr, (const int*)ids.ptr, hid.ptr, T, a.top, W, a.expert_ff, a.expert_act, a.act_limit,
                                             a.act_slope, f32, st),
                           "experts up"))
    return false;
  if (grouped == -2 &&
      !rc(k.pk_moe_down_combine(hid.ptr, L.e_down.d.ptr, (const int*)ids.ptr, (const float*)wts.ptr, shared, shared_gate, (float*)yf.ptr, T,
                                a.top, W, a.expert_ff, f32, st),
          "experts down"))
    return false;
  return true;
}

// Parallel block: on entry xa / h32 hold dyt(x) of this layer; on exit mix (element type) and, with a feed-forward, yf (fp32) hold the
// two sublayers' outputs -- the caller adds them to the residual together with the next norm.
bool Model::run_parallel_layer(int li, int T, const int* M, int n) {
  Layer& L = layers[li];
  const LayerCfg& a = L.c;
  const int f32 = c.f32, H = a.heads, G = a.kv_heads, mk = a.mixer_kind;
  const int *d_pos = M + T, *d_req = M + 2 * T, *d_poff = M + 3 * T, *d_slot = M + 3 * T + n, *d_row0 = M + 3 * T + 2 * n, *d_len = M + 3 * T + 3 * n;
  const int* d_pages = M + pages_at;
  const int nq = (mk == 2 ? G : H) * a.dim, nk = G * a.dim, nv = (mk == 1 ? G : H) * a.vdim, ng = mk == 1 ? 0 : H * a.vdim;
  const int nbig = nq + nk + nv + ng, E0 = a.mlp_kind == 2 ? a.experts : 0, nsmall = E0 + (mk >= 2 ? 2 * H : 0);
  if (!lin(L.qkv, xa.ptr, big.ptr, T)) return false;
  if (nsmall > 0 && !skinny(L.small, (float*)zs.ptr, T, "few-row projections", (const float*)h32.ptr)) return false;
  float* slot0 = state.ptr ? (float*)state.ptr + L.state_off : nullptr;
  if (mk == 1) {
    char* pool_base = (char*)cache.ptr + (size_t)L.cache_off * es;
    if (!rc(k.pk_gqa_rope_append(big.ptr, nbig, L.qkv_bias.d.ptr, d_pos, d_req, d_poff, d_pages, q.ptr, pool_base, page_stride, c.page_size, H, G, a.dim,
                                 a.vdim, a.rot_dims, a.rot_interleaved, (const float*)L.freq.ptr, L.mag, T, f32, st),
            "rotation + cache append"))
      return false;
    if (!rc(k.pk_gqa_attention(q.ptr, pool_base, L.sink.d.ptr, d_pos, d_req, d_poff, d_pages, ao.ptr, page_stride, c.page_size, T, H, G, a.dim, a.vdim,
                               a.scale, a.chunk, f32, st),
            "attention"))
      return false;
  } else if (mk == 2) {
    const int C = nq + nk + nv;
    if (!rc(k.pk_causal_conv_silu(big.ptr, nbig, L.conv_w.d.ptr, slot0 + (size_t)H * a.dim * a.vdim, slot_stride, d_req, d_slot, d_row0, d_len, convo.ptr, C, C,
                                  a.conv, T, n, f32, st),
            "short convolution"))
      return false;
    if (!rc(k.pk_gated_delta_seq(convo.ptr, C, 0, nq, nq + nk, (const float*)zs.ptr, nsmall, E0, E0 + H, (const float*)L.p0_32.ptr, (const float*)L.p1_32.ptr,
                                 slot0, slot_stride, d_slot, d_row0, d_len, (float*)orec.ptr, H, G, a.dim, a.vdim, n, f32, st),
            "gated delta rule"))
      return false;
    if (!rc(k.pk_head_norm_gate((const float*)orec.ptr, nullptr, L.hnorm.d.ptr, 0, big.ptr, nbig, nq + nk + nv, ao.ptr, T, H, a.vdim, c.eps, 0, f32, st),
            "read-out norm"))
      return false;
  } else {
    if (!rc(k.pk_mlstm_seq(big.ptr, nbig, 0, nq, nq + nk, (const float*)zs.ptr, nsmall, E0, E0 + H, (const float*)L.p0_32.ptr, (const float*)L.p1_32.ptr,
                           a.gate_cap, slot0, slot_stride, d_slot, d_row0, d_len, (float*)orec.ptr, (float*)den.ptr, H, a.dim, a.vdim, n, f32, st),
            "matrix memory"))
      return false;
    if (!rc(k.pk_head_norm_gate((const float*)orec.ptr, (const float*)den.ptr, L.hnorm.d.ptr, a.vdim, big.ptr, nbig, nq + nk + nv, ao.ptr, T, H, a.vdim,
                                c.eps, 1, f32, st),
            "read-out norm"))
      return false;
  }
  if (!lin(L.o, ao.ptr, mix.ptr, T)) return false;
  if (a.mlp_kind == 2) {
    if (!rc(k.pk_router_topk_ex((const float*)zs.ptr, nsmall, (const float*)L.corr32.ptr, (int*)ids.ptr, (float*)wts.ptr, T, a.experts, a.top, a.groups,
                                a.keep, a.route_scale, a.router_kind, a.router_kind == 1 ? 2 : 1, a.router_kind == 1 ? 0 : 1, st),
            "router top-k"))
      return false;
    if (!run_experts(L, T, nullptr, nullptr)) return false;
  }
  return true;
}

// One projection whose output rows fall into up to three segments, each written to its own packed buffer [N, seg_rows[i]]
bool Model::lin_segments(const Mat& W, const void* X, void* const* Y, const int* seg_rows, int N) {
  if (!c.f32 && N > 4) {
    pk_bf16* ys[3] = {(pk_bf16*)Y[0], (pk_bf16*)Y[1], (pk_bf16*)Y[2]};
    return rc(k.pk_b200_gemm_segments((const pk_bf16*)W.d.ptr, (const pk_bf16*)X, ys, seg_rows, W.rows, N, W.cols, st), "stacked projection");
  }
  if (!c.f32) {  // streaming GEMV with segmented output; shapes it does not take run one GEMV per segment below
    pk_b200_gemv_args g{};
    g.W = (const pk_bf16*)W.d.ptr;
    g.X = (const pk_bf16*)X;
    for (int i = 0; i < 3; ++i) {
      g.Y[i] = (pk_bf16*)Y[i];
      g.seg_rows[i] = seg_rows[i];
    }
    g.M = W.rows;
    g.N = N;
    g.K = W.cols;
    if (k.pk_b200_gemv_fused(&g, st) == 0) return true;
  }
  int r0 = 0;
  for (int i = 0; i < 3; ++i) {
    if (seg_rows[i] <= 0) continue;
    const char* base = (const char*)W.d.ptr + (size_t)r0 * W.cols * es;
    if (c.f32) {
      if (!rc(k.pk_gemm_strided(X, base, Y[i], nullptr, N, seg_rows[i], W.cols, W.cols, 1, W.cols, seg_rows[i], 1, 0, 0, 0, 0, 0, 1, st), "stacked projection"))
        return false;
    } else {
      k.gemm_cuda((const pk_bf16*)base, (const pk_bf16*)X, (pk_bf16*)Y[i], seg_rows[i], N, W.cols, st);
    }
    r0 += seg_rows[i];
  }
  return true;
}

// Sandwich block: on entry xa holds gnorm(x, norm1) of this layer; on exit x holds the layer's result and xa the next layer's
// pre-norm (nothing after the last layer).
bool Model::run_sandwich_layer(int li, int T, int max_kv, const int* M) {
  Layer& L = layers[li];
  const LayerCfg& a = L.c;
  const int W = c.width, f32 = c.f32, H = a.heads, G = a.kv_heads, mk = a.mixer_kind, rg = c.gated_residual ? W : 0;
  const int *d_pos = M + T, *d_req = M + 2 * T, *d_poff = M + 3 * T;
  const int* d_pages = M + pages_at;
  char* pool_base = (char*)cache.ptr + (size_t)L.cache_off * es;
  const void* sink = a.sink_kind == 0 ? L.sink.d.ptr : a.sink_kind == 2 ? zero_sink.ptr : nullptr;
  const void* gate1 = nullptr;  // pre-activation of the gate on the mixer's result
  long gate1_ld = 0;
  if (mk == 1) {
    const int nq = H * a.dim, nk = G * a.dim, nv = G * a.vdim, ng = a.out_gate ? H * a.vdim : 0, nbig = nq + nk + nv + ng + rg;
    if (!lin(L.qkv, xa.ptr, big.ptr, T)) return false;
    if (!rc(k.pk_gqa_rope_append_ex(big.ptr, nbig, L.qkv_bias.d.ptr, d_pos, d_req, d_poff, d_pages, q.ptr, pool_base, page_stride, c.page_size, H, G, a.dim,
                                    a.vdim, a.rot_dims, a.rot_interleaved, (const float*)L.freq.ptr, L.mag, a.value_norm ? c.eps : 0.f, T, f32, st),
            "cache append"))
      return false;
    pk_attn_extra ex{};
    ex.window = a.window;
    ex.softcap = a.softcap;
    ex.slope_log2 = a.slope_log2;
    ex.gate = ng ? (const char*)big.ptr + (size_t)(nq + nk + nv) * es : nullptr;
    ex.gate_ld = nbig;
    ex.max_kv_len = max_kv;
    if (!rc(k.pk_gqa_attention_ex(q.ptr, pool_base, sink, d_pos, d_req, d_poff, d_pages, ao.ptr, page_stride, c.page_size, T, H, G, a.dim, a.vdim, a.scale,
                                  a.chunk, &ex, f32, st),
            "attention"))
      return false;
    if (rg) {
      gate1 = (const char*)big.ptr + (size_t)(nq + nk + nv + ng) * es;
      gate1_ld = nbig;
    }
  } else {
    const int r = a.kv_rank, rd = a.rot_dim, D = r + rd;
    void* outs[3] = {q.ptr, dkv.ptr, rgbuf.ptr};
    const int segs[3] = {H * (a.dim + rd), D, rg};
    if (!lin_segments(L.qkv, xa.ptr, outs, segs, T)) return false;
    if (!rc(k.pk_latent_kv_append_ex(dkv.ptr, L.dkv_norm.d.ptr, d_pos, d_req, d_poff, d_pages, pool_base, page_stride, c.page_size, r, rd, a.rot_dims,
                                     a.rot_interleaved, (const float*)L.freq.ptr, L.mag, c.eps, T, f32, st),
            "latent cache append"))
      return false;
    // fold the unrotated query onto the latent (per head: qa[:, :r] = q_unrotated W_uk[h]), rotate the other part beside it
    if (!rc(k.pk_gemm_strided(q.ptr, L.uk_t.d.ptr, qa.ptr, nullptr, T, r, a.dim, (long)H * (a.dim + rd), 1, a.dim, (long)H * D, H, a.dim + rd,
                              (long)a.dim * r, D, 0, 0, f32, st),
            "query fold"))
      return false;
    if (rd > 0 && !rc(k.pk_rope_slice_ex(q.ptr, qa.ptr, d_pos, (const float*)L.freq.ptr, L.mag, T, H, a.dim + rd, a.dim, D, r, rd, a.rot_dims, a.rot_interleaved,
                                         f32, st),
                      "query rotation"))
      return false;
    if (!rc(k.pk_latent_attention_ex(qa.ptr, pool_base, sink, d_pos, d_req, d_poff, d_pages, olat.ptr, page_stride, c.page_size, T, H, r, rd, a.scale, a.window,
                                     max_kv, f32, st),
            "latent attention"))
      return false;
    if (!rc(k.pk_gemm_strided(olat.ptr, L.uv.d.ptr, ao.ptr, nullptr, T, a.vdim, r, (long)H * r, 1, r, (long)H * a.vdim, H, r, (long)a.vdim * r, a.vdim, 0, 0, f32,
                              st),
            "value expansion"))
      return false;
    if (rg) {
      gate1 = rgbuf.ptr;
      gate1_ld = W;
    }
  }
  if (!lin(L.o, ao.ptr, mix.ptr, T)) return false;
  const Layer* next = li + 1 < c.n_layers ? &layers[li + 1] : nullptr;
  const void* after_mixer = a.mlp_kind ? L.norm2.d.ptr : next ? next->norm1.d.ptr : nullptr;
  if (!rc(k.pk_res32_gated_gnorm_add(mix.ptr, f32, L.o_bias.d.ptr, gate1, gate1_ld, gate1 ? L.rg1_bias.d.ptr : nullptr, L.norm1b.d.ptr, c.residual_mult,
                                     (float*)x.ptr, after_mixer, xa.ptr, W, c.norm_groups, c.eps, T, f32, st),
          "mixer result: gate, norm, residual"))
    return false;
  if (a.mlp_kind == 1) {
    // gate | up projection with the SwiGLU activation in its epilogue where the library has it (as in the sequential block)
    bool fused = false;
    if (!f32 && T <= 4) {
      pk_b200_gemv_args g{};
      g.W = (const pk_bf16*)L.gate_up.d.ptr;
      g.X = (const pk_bf16*)xa.ptr;
      g.Y[0] = (pk_bf16*)act.ptr;
      g.seg_rows[0] = a.ff;
      g.M = a.ff;
      g.N = T;
      g.K = W;
      g.epi = 1;
      fused = k.pk_b200_gemv_fused(&g, st) == 0;
    } else if (!f32) {
      fused = k.pk_b200_gemm_swiglu((const pk_bf16*)L.gate_up.d.ptr, (const pk_bf16*)xa.ptr, (pk_bf16*)act.ptr, a.ff, T, W, st) == 0;
    }
    if (!fused) {
      if (!lin(L.gate_up, xa.ptr, gu.ptr, T)) return false;
      if (!rc(k.pk_act(gu.ptr, act.ptr, a.ff, T, 0, f32, st), "SwiGLU")) return false;
    }
    if (rg && !lin(L.rg2, xa.ptr, rgbuf.ptr, T)) return false;
    if (!lin(L.down, act.ptr, mix.ptr, T)) return false;
    if (!rc(k.pk_res32_gated_gnorm_add(mix.ptr, f32, nullptr, rg ? rgbuf.ptr : nullptr, W, rg ? L.rg2_bias.d.ptr : nullptr, L.norm2b.d.ptr, c.residual_mult,
                                       (float*)x.ptr, next ? next->norm1.d.ptr : nullptr, xa.ptr, W, c.norm_groups, c.eps, T, f32, st),
            "feed-forward result: gate, norm, residual"))
      return false;
  }
  if (keep_trail)
    return cu(cudaMemcpyAsync((char*)trail.ptr + (size_t)li * T * W * 4, x.ptr, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, st), "trail copy");
  return true;
}

// Pre-norm block: on entry xa (and h32, unrounded) hold rms(x) * norm1 of this layer; on exit x holds the layer's result and xa / h32
// the next layer's pre-norm (nothing after the last layer).  Weights come from layer `wsrc`, cache and state are this layer's own.
bool Model::run_prenorm_layer(int li, int T, int max_kv, const int* M, int n) {
  Layer& L = layers[li];
  const Layer& Wt = layers[L.wsrc];
  const LayerCfg& a = L.c;
  const int W = c.width, f32 = c.f32, H = a.heads, G = a.kv_heads, mk = a.mixer_kind;
  const int *d_pos = M + T, *d_req = M + 2 * T, *d_poff = M + 3 * T, *d_slot = M + 3 * T + n, *d_row0 = M + 3 * T + 2 * n, *d_len = M + 3 * T + 3 * n;
  const int* d_pages = M + pages_at;
  char* pool_base = (char*)cache.ptr + (size_t)L.cache_off * es;
  const int nq = H * a.dim, nk = G * a.dim, nv = mk == 1 && !a.values_are_keys ? G * a.vdim : 0;
  const int inner = mk == 4 ? a.ssm_heads * a.ssm_vdim : 0, C = mk == 4 ? inner + 2 * a.ssm_groups * a.ssm_state : 0;
  const int nin = mk == 4 ? inner + C + a.ssm_heads : 0, nbig = nq + nk + nv + nin;
  const Layer* next = li + 1 < c.n_layers ? &layers[layers[li + 1].wsrc] : nullptr;
  const void* after_mixer = a.mlp_kind ? Wt.norm2.d.ptr : next ? next->norm1.d.ptr : nullptr;
  // ---- mixer: one stacked projection, then the attention (both mixers have one)
  if (!lin(Wt.qkv, xa.ptr, big.ptr, T)) return false;
  pk_qk_prep prep{};
  prep.norm_kind = a.qk_norm;
  prep.q_weight = Wt.qn.d.ptr;
  prep.k_weight = Wt.kn.d.ptr;
  prep.eps = c.eps;
  prep.temp_coef = a.q_temp_coef;
  prep.temp_every = a.q_temp_every;
  prep.values_are_keys = a.values_are_keys;
  if (!rc(k.pk_gqa_norm_append(big.ptr, nbig, d_pos, d_req, d_poff, d_pages, q.ptr, pool_base, page_stride, c.page_size, H, G, a.dim, a.vdim, a.rot_dims,
                               a.rot_interleaved, (const float*)Wt.freq.ptr, Wt.mag, &prep, T, f32, st),
          "q / k norm + cache append"))
    return false;
  pk_attn_extra ex{};
  ex.window = a.window;
  ex.keep_first = a.keep_first;
  ex.max_kv_len = max_kv;
  if (!rc(k.pk_gqa_attention_ex(q.ptr, pool_base, a.sink_kind == 0 ? Wt.sink.d.ptr : nullptr, d_pos, d_req, d_poff, d_pages, ao.ptr, page_stride, c.page_size,
                                T, H, G, a.dim, a.vdim, a.scale, a.chunk, &ex, f32, st),
          "attention"))
    return false;
  if (!lin(Wt.o, ao.ptr, mix.ptr, T)) return false;
  if (mk == 4) {
    // ---- state-space branch on the rows [z | x B C | dt] of the same projection
    const int in_off = nq + nk, Hs = a.ssm_heads, N = a.ssm_state, P = a.ssm_vdim, gs = inner / a.ssm_norm_groups;
    float* slot0 = (float*)state.ptr + L.state_off;
    if (!rc(k.pk_causal_conv_silu_bias((const char*)big.ptr + (size_t)(in_off + inner) * es, nbig, Wt.conv_w.d.ptr, Wt.conv_b.d.ptr,
                                       slot0 + (size_t)Hs * N * P, slot_stride, d_req, d_slot, d_row0, d_len, convo.ptr, C, C, a.conv, T, n, f32, st),
            "short convolution"))
      return false;
    if (!rc(k.pk_ssd_seq(convo.ptr, C, 0, inner, inner + a.ssm_groups * N, big.ptr, nbig, in_off + inner + C, (const float*)Wt.p0_32.ptr,
                         (const float*)Wt.p1_32.ptr, (const float*)Wt.p2_32.ptr, slot0, slot_stride, d_slot, d_row0, d_len, (float*)orec.ptr, Hs,
                         a.ssm_groups, N, P, n, f32, st),
            "state-space recurrence"))
      return false;
    if (!rc(k.pk_head_norm_gate((const float*)orec.ptr, nullptr, Wt.hnorm.d.ptr, gs, big.ptr, nbig, in_off, ao2.ptr, T, a.ssm_norm_groups, gs, c.eps, 2, f32,
                                st),
            "gated read-out norm"))
      return false;
    if (!lin(Wt.o2, ao2.ptr, mix2.ptr, T)) return false;
    if (!rc(k.pk_res32_branches_add_norm(mix.ptr, 0, Wt.lout.d.ptr, mix2.ptr, Wt.rout.d.ptr, 0.5f, (float*)x.ptr, after_mixer, xa.ptr, (float*)h32.ptr, W,
                                         c.eps, T, f32, st),
            "mixer result: branch norms, residual, next norm"))
      return false;
  } else if (!rc(k.pk_res32_branches_add_norm(mix.ptr, 0, nullptr, nullptr, nullptr, 1.f, (float*)x.ptr, after_mixer, xa.ptr, (float*)h32.ptr, W, c.eps, T,
                                              f32, st),
                 "mixer result: residual, next norm")) {
    return false;
  }
  // ---- feed-forward: routed experts plus an ungated shared expert of the same form
  if (a.mlp_kind == 2) {
    if (!skinny(Wt.router, (float*)z.ptr, T, "router", (const float*)h32.ptr)) return false;
    if (!rc(k.pk_router_topk_logits((const float*)z.ptr, a.experts, (const float*)Wt.corr32.ptr, (int*)ids.ptr, (float*)wts.ptr, T, a.experts, a.top,
                                    a.route_scale, st),
            "router top-k"))
      return false;
    const void* shared = nullptr;
    if (a.shared_ff > 0) {
      if (!lin(Wt.gate_up, xa.ptr, gu.ptr, T)) return false;
      if (!rc(k.pk_act_clamped(gu.ptr, act.ptr, a.shared_ff, T, a.shared_limit, a.act_slope, f32, st), "shared expert activation")) return false;
      if (!lin(Wt.s_down, act.ptr, sh.ptr, T)) return false;
      shared = sh.ptr;
    }
    if (!run_experts(Wt, T, shared, nullptr)) return false;
    if (!rc(k.pk_res32_branches_add_norm(yf.ptr, 1, nullptr, nullptr, nullptr, 1.f, (float*)x.ptr, next ? next->norm1.d.ptr : nullptr, xa.ptr,
                                         (float*)h32.ptr, W, c.eps, T, f32, st),
            "feed-forward result: residual, next norm"))
      return false;
  }
  if (keep_trail)
    return cu(cudaMemcpyAsync((char*)trail.ptr + (size_t)li * T * W * 4, x.ptr, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, st), "trail copy");
  return true;
}

// everything between the metadata upload and the final synchronisation: launches only (no allocation, no synchronisation)
bool Model::forward(int T, int n, int n_rows, int max_kv, int want_sample) {
  const int* M = meta_d.i32();
  const int *d_tok = M, *d_pos = M + T, *d_req = M + 2 * T, *d_poff = M + 3 * T, *d_rows = M + 3 * T + 4 * n, *d_pages = M + 3 * T + 4 * n + n_rows;
  pages_at = 3 * T + 4 * n + n_rows;
  const int W = c.width;
  if (c.block_kind == 0) {
    if (!rc(k.pk_res32_embed(embed.d.ptr, d_tok, (float*)x.ptr, xa.ptr, W, T, c.f32, st), "embedding")) return false;
    for (int li = 0; li < c.n_layers; ++li)
      if (!run_layer(li, T, max_kv, d_pos, d_req, d_poff, d_pages)) return false;
  } else if (c.block_kind == 3) {
    if (!rc(k.pk_res32_embed_scaled_norm(embed.d.ptr, d_tok, c.embed_scale, (float*)x.ptr, layers[layers[0].wsrc].norm1.d.ptr, xa.ptr, (float*)h32.ptr, W, c.eps,
                                         T, c.f32, st),
            "embedding"))
      return false;
    for (int li = 0; li < c.n_layers; ++li)
      if (!run_prenorm_layer(li, T, max_kv, M, n)) return false;
  } else if (c.block_kind == 2) {
    if (!rc(k.pk_res32_embed_gnorm(embed.d.ptr, d_tok, embed_norm.d.ptr, (float*)x.ptr, layers[0].norm1.d.ptr, xa.ptr, W, c.norm_groups, c.eps, T, c.f32, st),
            "embedding"))
      return false;
    for (int li = 0; li < c.n_layers; ++li)
      if (!run_sandwich_layer(li, T, max_kv, M)) return false;
  } else {
    if (!rc(k.pk_res32_embed_scaled(embed.d.ptr, d_tok, (float*)x.ptr, W, T, c.embed_scale, c.f32, st), "embedding")) return false;
    // every layer's residual sum is folded into the next layer's norm (the last one into a plain sum)
    for (int li = 0; li <= c.n_layers; ++li) {
      const Layer* P = li > 0 ? &layers[li - 1] : nullptr;
      const Layer* N = li < c.n_layers ? &layers[li] : nullptr;
      if (!rc(k.pk_res32_add_dyt(P ? mix.ptr : nullptr, P && P->c.mlp_kind == 2 ? (const float*)yf.ptr : nullptr, N ? (const float*)N->alpha32.ptr : nullptr,
                                 N ? N->norm1.d.ptr : nullptr, N ? N->nb.d.ptr : nullptr, (float*)x.ptr, xa.ptr, (float*)h32.ptr, W, T, c.f32, st),
              "residual sum + norm"))
        return false;
      if (keep_trail && P &&
          !cu(cudaMemcpyAsync((char*)trail.ptr + (size_t)(li - 1) * T * W * 4, x.ptr, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, st), "trail copy"))
        return false;
      if (N && !run_parallel_layer(li, T, M, n)) return false;
    }
  }
  if (n_rows > 0) {
    if (c.block_kind == 0) {
      if (!rc(k.pk_res32_offset_norm_rows((const float*)x.ptr, d_rows, final_norm.d.ptr, xr.ptr, W, n_rows, c.eps, c.f32, st), "final norm")) return false;
    } else if (c.block_kind >= 2) {  // the pre-norm block form's last norm is the same norm with one group
      if (!rc(k.pk_res32_gnorm_rows((const float*)x.ptr, d_rows, final_norm.d.ptr, xr.ptr, W, c.block_kind == 2 ? c.norm_groups : 1, c.eps, n_rows, c.f32, st),
              "final norm"))
        return false;
    } else if (!rc(k.pk_res32_dyt_rows((const float*)x.ptr, d_rows, (const float*)final_alpha32.ptr, final_norm.d.ptr, final_b.d.ptr, xr.ptr, W, n_rows, c.f32,
                                       st),
                   "final norm")) {
      return false;
    }
    if (!lin(head, xr.ptr, logits_e.ptr, n_rows)) return false;
    const float ls = c.block_kind >= 1 ? c.logit_scale : 1.f;
    if (c.block_kind == 3) {
      if (!rc(k.pk_logits_scale_cap(logits_e.ptr, c.f32, (float*)logits_f.ptr, (long)n_rows * c.vocab, ls, c.logit_softcap, st), "logits")) return false;
    } else if (!rc(k.pk_scale_to_f32(logits_e.ptr, c.f32, (float*)logits_f.ptr, (long)n_rows * c.vocab, ls, st), "logits")) {
      return false;
    }
    if (want_sample) {
      if (c.f32 || ls != 1.f || c.block_kind == 3) {  // the final (scaled) logits exist in fp32 only: greedy token of every row from those
        if (!rc(k.pk_top1_rows_f32((const float*)logits_f.ptr, sampled_d.i32(), n_rows, c.vocab, st), "greedy token")) return false;
      } else {
        const pk_bf16* lb = (const pk_bf16*)logits_e.ptr;
        for (int i = 0; i < n_rows; ++i)
          k.flashinfer_top1_cuda(lb + (size_t)i * c.vocab, (pk_bf16*)top1_val.ptr, (uint8_t*)top1_states.ptr, sampled_d.i32() + i, c.vocab, st);
      }
      if (!cu(cudaMemcpyAsync(sampled_h, sampled_d.ptr, (size_t)std::min(n_rows, 1024) * 4, cudaMemcpyDeviceToHost, st), "sampled tokens")) return false;
    }
  }
  return true;
}

// One engine step over a ragged batch.  tokens: all entries' tokens back to back; lens[i] tokens belong to request rids[i];
// rows: indices into that flat token list whose logits are wanted.  Leaves fp32 logits [n_rows, vocab] in logits_f (and the
// greedy token of each row in sampled_h when want_sample).
bool Model::step(int n, const int* tokens, const int* lens, const int* rids, int n_rows, const int* rows, int want_sample) {
  if (!finalized) return fail("model not finalized");
  if (n <= 0) return fail("empty step");
  int T = 0, pages_needed = 0;
  for (int i = 0; i < n; ++i) {
    if (rids[i] < 0 || rids[i] >= (int)reqs.size() || !reqs[rids[i]].live) return fail("bad request id");
    for (int j = 0; j < i; ++j)
      if (rids[j] == rids[i]) return fail("a request appears twice in one step");
    if (lens[i] <= 0) return fail("an entry without tokens");
    const pq::KvState& s = reqs[rids[i]];
    pages_needed += std::max(0, (s.seq_len + lens[i] + c.page_size - 1) / c.page_size - (int)s.pages.size());
    T += lens[i];
  }
  for (int t = 0; t < T; ++t)
    if (tokens[t] < 0 || tokens[t] >= c.vocab) return fail("token id outside the vocabulary");
  for (int i = 0; i < n_rows; ++i)
    if (rows[i] < 0 || rows[i] >= T) return fail("logits row outside the step");
  if (pages_needed > (int)pool.free_list.size()) {
    char b[128];
    snprintf(b, sizeof b, "cache pool: out of pages (need %d more, %d available)", pages_needed, (int)pool.free_list.size());
    return fail(b);
  }
  if (!ensure_scratch(T, std::max(n_rows, 1))) return false;
  if (keep_trail && !trail.alloc_uninit((size_t)c.n_layers * T * c.width * 4)) return fail("trail allocation failed");
  trail_tokens = T;
  struct Txn {  // undo record: a failure below gives back the pages and the lengths of this step
    Model* m;
    std::vector<std::pair<int, std::pair<int, size_t>>> old;
    bool committed = false;
    ~Txn() {
      if (committed) return;
      for (auto& o : old) {
        pq::KvState& s = m->reqs[o.first];
        std::vector<int> extra(s.pages.begin() + o.second.second, s.pages.end());
        m->pool.release(extra);
        s.pages.resize(o.second.second);
        s.seq_len = o.second.first;
      }
    }
  } txn{this, {}, false};
  // metadata block: [tok T][pos T][req T][page_off n][slot n][row0 n][len n][rows R][pages ...]
  std::vector<int> meta((size_t)3 * T + 4 * n + n_rows);
  int t0 = 0, max_kv = 0;
  std::vector<int> page_list;
  for (int i = 0; i < n; ++i) {
    pq::KvState& s = reqs[rids[i]];
    txn.old.push_back({rids[i], {s.seq_len, s.pages.size()}});
    const int need = (s.seq_len + lens[i] + c.page_size - 1) / c.page_size - (int)s.pages.size();
    if (need > 0 && !pool.acquire(need, &s.pages)) return fail("cache pool: out of pages");
    for (int t = 0; t < lens[i]; ++t) {
      meta[t0 + t] = tokens[t0 + t];
      meta[T + t0 + t] = s.seq_len + t;
      meta[2 * T + t0 + t] = i;
    }
    meta[3 * T + i] = (int)page_list.size();
    meta[3 * T + n + i] = rids[i];
    meta[3 * T + 2 * n + i] = t0;
    meta[3 * T + 3 * n + i] = lens[i];
    if (fresh[rids[i]] && state.ptr) {  // a slot that another request used before: its state starts at zero
      if (!cu(cudaMemsetAsync((float*)state.ptr + (size_t)rids[i] * slot_stride, 0, (size_t)slot_stride * 4, st), "state reset")) return false;
    }
    fresh[rids[i]] = 0;
    page_list.insert(page_list.end(), s.pages.begin(), s.pages.end());
    s.seq_len += lens[i];
    max_kv = std::max(max_kv, s.seq_len);
    t0 += lens[i];
  }
  for (int i = 0; i < n_rows; ++i) meta[3 * T + 4 * n + i] = rows[i];
  meta.insert(meta.end(), page_list.begin(), page_list.end());
  if (meta.size() > meta_cap) {
    cudaStreamSynchronize(st);
    drop_graphs();
    if (meta_h) cudaFreeHost(meta_h);
    meta_cap = meta.size() * 2 + 1024;
    if (cudaMallocHost((void**)&meta_h, meta_cap * 4) != cudaSuccess || !meta_d.alloc_uninit(meta_cap * 4)) {
      meta_h = nullptr;
      meta_cap = 0;
      return fail("metadata allocation failed");
    }
  }
  memcpy(meta_h, meta.data(), meta.size() * 4);
  if (!cu(cudaMemcpyAsync(meta_d.ptr, meta_h, meta.size() * 4, cudaMemcpyHostToDevice, st), "metadata upload")) return false;
  // Decode steps (one token per entry) repeat with the same shapes: the launch sequence is captured once per (entries, rows,
  // sampling, context bucket) and replayed; only the metadata block changes.  The first step of a kind runs eagerly (it also
  // lets every kernel set its attributes outside a capture).
  bool single = use_graph && !keep_trail && T == n;
  bool ok;
  if (single) {
    const int bucket = (max_kv + kGraphCtxBucket - 1) / kGraphCtxBucket;
    const GraphKey key{n, n_rows, want_sample, bucket};
    auto it = graphs.find(key);
    if (it != graphs.end()) {
      ok = cu(cudaGraphLaunch(it->second, st), "graph launch");
    } else if (seen.count(key)) {
      ok = cu(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal), "begin capture");
      if (ok) {
        const bool body_ok = forward(T, n, n_rows, bucket * kGraphCtxBucket, want_sample);
        cudaGraph_t gr = nullptr;
        const cudaError_t e = cudaStreamEndCapture(st, &gr);
        cudaGraphExec_t ex = nullptr;
        ok = body_ok && cu(e, "end capture") && cu(cudaGraphInstantiate(&ex, gr, 0), "graph instantiate");
        if (gr) cudaGraphDestroy(gr);
        if (ok) {
          graphs[key] = ex;
          ok = cu(cudaGraphLaunch(ex, st), "graph launch");
        }
      }
    } else {
      seen.insert(key);
      ok = forward(T, n, n_rows, bucket * kGraphCtxBucket, want_sample);
    }
  } else {
    ok = forward(T, n, n_rows, max_kv, want_sample);
  }
  if (!ok) return false;
  if (!cu(cudaStreamSynchronize(st), "step")) return false;
  txn.committed = true;
  return true;
}

}  // namespace pv

extern "C" {

static thread_local std::string g_pv_err;
#define PV_API __attribute__((visibility("default")))
#define PV_M static_cast<pv::Model*>(mp)

PV_API const char* pv_create_error() { return g_pv_err.c_str(); }

PV_API void* pv_create(const pv::ModelCfg* mc, const pv::LayerCfg* lc, const char* kernel_lib_path) {
  auto* m = new pv::Model();
  auto bail = [&](const std::string& e) -> void* {
    g_pv_err = e;
    delete m;
    return nullptr;
  };
  if (!m->configure(*mc, lc)) return bail(m->err);
  std::string e = m->k.load(kernel_lib_path, mc->block_kind);
  if (!e.empty()) return bail(e);
  if (m->k.cuda_set_device(mc->device) != 0) return bail("cuda_set_device failed (no CUDA device?)");
  if (cudaStreamCreateWithFlags(&m->st, cudaStreamNonBlocking) != cudaSuccess)
    return bail(std::string("stream creation failed: ") + cudaGetErrorString(cudaGetLastError()));
  m->k.cublas_init();
  m->k.pk_b200_set_pdl(mc->enable_pdl);
  g_pv_err.clear();
  return m;
}
PV_API void pv_destroy(void* mp) { delete PV_M; }
PV_API const char* pv_last_error(void* mp) { return PV_M->err.c_str(); }
PV_API int pv_load_tensor(void* mp, const char* name, const void* data, int rows, int cols, int is_f32) {
  return PV_M->load_tensor(name, data, rows, cols, is_f32) ? 0 : -1;
}
PV_API int pv_finalize(void* mp) { return PV_M->finalize() ? 0 : -1; }
PV_API int pv_request_alloc(void* mp) {
  auto& v = PV_M->reqs;
  for (size_t i = 0; i < v.size(); ++i)
    if (!v[i].live) {
      v[i] = pq::KvState();
      v[i].live = true;
      PV_M->fresh[i] = 1;
      return (int)i;
    }
  PV_M->err = "every request slot is in use";
  return -1;
}
PV_API void pv_request_free(void* mp, int id) {
  auto& v = PV_M->reqs;
  if (id < 0 || id >= (int)v.size() || !v[id].live) return;
  PV_M->pool.release(v[id].pages);
  v[id] = pq::KvState();
}
PV_API int pv_seq_len(void* mp, int id) {
  auto& v = PV_M->reqs;
  return (id < 0 || id >= (int)v.size() || !v[id].live) ? -1 : v[id].seq_len;
}
PV_API int pv_available_pages(void* mp) { return (int)PV_M->pool.free_list.size(); }
PV_API int pv_page_size(void* mp) { return PV_M->c.page_size; }
// the pages a request holds, in order (tests check that freed pages are handed out again)
PV_API int pv_request_pages(void* mp, int id, int* out, int cap) {
  auto& v = PV_M->reqs;
  if (id < 0 || id >= (int)v.size() || !v[id].live) return -1;
  const int n = (int)v[id].pages.size();
  for (int i = 0; i < std::min(n, cap); ++i) out[i] = v[id].pages[i];
  return n;
}
PV_API int pv_step(void* mp, int n, const int* tokens, const int* lens, const int* rids, int n_rows, const int* rows, int want_sample,
                   float* logits_host, int* sampled) {
  pv::Model* m = PV_M;
  if (!m->step(n, tokens, lens, rids, n_rows, rows, want_sample)) return -1;
  if (n_rows > 0 && logits_host &&
      cudaMemcpy(logits_host, m->logits_f.ptr, (size_t)n_rows * m->c.vocab * 4, cudaMemcpyDeviceToHost) != cudaSuccess) {
    m->err = "logits copy failed";
    return -1;
  }
  if (want_sample && sampled)
    for (int i = 0; i < std::min(n_rows, 1024); ++i) sampled[i] = m->sampled_h[i];
  return 0;
}
PV_API void pv_keep_trail(void* mp, int on) { PV_M->keep_trail = on != 0; }
PV_API void pv_use_graph(void* mp, int on) { PV_M->use_graph = on != 0; }
PV_API int pv_graph_count(void* mp) { return (int)PV_M->graphs.size(); }
// residual stream after every layer of the last step, [layers, tokens, width] fp32
PV_API int pv_copy_trail(void* mp, float* host_out) {
  pv::Model* m = PV_M;
  if (!m->keep_trail || !m->trail.ptr) return -1;
  return cudaMemcpy(host_out, m->trail.ptr, (size_t)m->c.n_layers * m->trail_tokens * m->c.width * 4, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -1;
}
PV_API int64_t pv_launch_count(void* mp, int reset) { return PV_M->k.pk_b200_launch_count(reset); }

// greedy generation of one request, timed like the other hosts' generate: first token after the whole prompt, then one step per token
PV_API int pv_generate(void* mp, const int* prompt, int n_prompt, int max_tokens, int* out, double* ttft_ms, double* step_ms) {
  pv::Model* m = PV_M;
  const int rid = pv_request_alloc(mp);
  if (rid < 0) return -1;
  using clk = std::chrono::steady_clock;
  auto t0 = clk::now();
  int row = n_prompt - 1, len = n_prompt, ok = 1;
  if (!m->step(1, prompt, &len, &rid, 1, &row, 1)) ok = 0;
  if (ok) {
    out[0] = m->sampled_h[0];
    *ttft_ms = std::chrono::duration<double, std::milli>(clk::now() - t0).count();
    for (int i = 1; i < max_tokens && ok; ++i) {
      auto t1 = clk::now();
      int one = 1, zero = 0, tok = out[i - 1];
      if (!m->step(1, &tok, &one, &rid, 1, &zero, 1)) ok = 0;
      else out[i] = m->sampled_h[0];
      step_ms[i - 1] = std::chrono::duration<double, std::milli>(clk::now() - t1).count();
    }
  }
  pv_request_free(mp, rid);
  return ok ? 0 : -1;
}
}
