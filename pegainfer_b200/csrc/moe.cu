// Mixture-of-experts feed-forward: group-limited top-k routing over softmax scores, and the chosen experts' two-matrix
// feed-forward (up -> activation -> down) gathered per token, plus an optional always-on shared expert that enters
// through a per-token logistic gate.
//   router: s = softmax(z) over all experts (fp32); experts are split into `groups` equal runs of neighbours, a group
//           scores as its best expert, only the `keep` best groups stay eligible; the `top` best eligible experts are
//           chosen (lowest index wins ties); weight = s / (sum of chosen s + 1e-20) * scale.
//   experts: hid[t,k,:] = act(W_up[e_k] x_t);  y[t] = sum_k w_k W_down[e_k] hid[t,k,:]  (+ logistic(g_t) * shared[t]).
//   Variants (parameters of the `_ex` / `_act` entry points): logistic scores instead of softmax, a per-expert correction added to
//   the scores for the CHOICE only (weights use the uncorrected score), a group scoring as the sum of its two best corrected
//   scores, weights not renormalised; experts with a gated activation, hid = silu(W_gate x) * (W_up x), whose gate and up rows
//   are stored interleaved (row 2f = gate f, row 2f + 1 = up f) so that one pass yields both; a gated activation with clamped
//   pre-activations, g = min(gate, limit), u = clamp(up, -limit, limit), hid = g * logistic(slope * g) * (u + 1); a router that picks
//   the largest logits (+ bias) and weighs the picked experts by the softmax over their logits alone; a shared expert without a gate.
// The per-token form reads only the chosen experts' weights: the decode path (a few tokens) is bound by those bytes.
#include "common.cuh"
#include "typed.cuh"

namespace pk {

// (value, index) arg-max over a warp, lowest index on ties
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) {
      v = ov;
      i = oi;
    }
  }
}

// one warp per token; shared memory: scores [E] + group eligibility [groups]
// score_kind 0: softmax over the experts, 1: logistic per expert.  corr (may be null): added to the score for choosing.
// score_kind 2: the score is the logit + corr (a bias that counts for choice AND weight); weights = softmax over the chosen scores.
// group_top 1: a group scores as its best expert, 2: as the sum of its two best.  renorm 1: weights divided by their sum.
__global__ void router_grouped_topk_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ corr, int* __restrict__ ids,
                                           float* __restrict__ wts, int E, int top, int groups, int keep, float scale, int score_kind, int group_top,
                                           int renorm) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x, lane = threadIdx.x;
  float* s = sm;            // [E] score (weight source)
  float* c = s + E;         // [E] choice score = score + correction; -inf once taken
  float* gs = c + E;        // [groups] group score, -inf once taken
  float* ok = gs + groups;  // [groups] 1 = eligible
  const float* zr = z + (size_t)t * ldz;
  if (score_kind == 0) {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zr[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float v = expf(zr[e] - mx);
      s[e] = v;
      sum += v;
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    __syncwarp();
    for (int e = lane; e < E; e += 32) s[e] *= inv;
  } else if (score_kind == 1) {
    for (int e = lane; e < E; e += 32) s[e] = 1.f / (1.f + expf(-zr[e]));
  } else {
    for (int e = lane; e < E; e += 32) s[e] = zr[e] + (corr ? corr[e] : 0.f);
  }
  __syncwarp();
  for (int e = lane; e < E; e += 32) c[e] = score_kind == 2 ? s[e] : s[e] + (corr ? corr[e] : 0.f);
  __syncwarp();
  const int per = E / groups;
  for (int g = lane; g < groups; g += 32) {
    float b1 = -INFINITY, b2 = -INFINITY;
    for (int e = 0; e < per; ++e) {
      const float v = c[g * per + e];
      if (v > b1) {
        b2 = b1;
        b1 = v;
      } else if (v > b2) {
        b2 = v;
      }
    }
    gs[g] = (group_top >= 2 && per >= 2) ? b1 + b2 : b1;
    ok[g] = 0.f;
  }
  __syncwarp();
  for (int r = 0; r < keep; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int g = lane; g < groups; g += 32)
      if (ok[g] == 0.f && (gs[g] > bv || bi == 0x7fffffff)) {
        bv = gs[g];
        bi = g;
      }
    warp_argmax(bv, bi);
    if (lane == 0) ok[bi] = 1.f;
    __syncwarp();
  }
  float total = 0.f;
  for (int r = 0; r < top; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (ok[e / per] > 0.f && c[e] != -INFINITY && (c[e] > bv || bi == 0x7fffffff)) {
        bv = c[e];
        bi = e;
      }
    warp_argmax(bv, bi);
    const float w = s[bi];
    total += w;
    if (lane == 0) {
      ids[(size_t)t * top + r] = bi;
      wts[(size_t)t * top + r] = w;
      c[bi] = -INFINITY;  // taken
    }
    __syncwarp();
  }
  __syncwarp();
  if (score_kind == 2) {  // the first pick carries the largest score
    const float mx = wts[(size_t)t * top];
    float sum = 0.f;
    for (int r = lane; r < top; r += 32) sum += expf(wts[(size_t)t * top + r] - mx);
    sum = warp_sum(sum);
    for (int r = lane; r < top; r += 32) wts[(size_t)t * top + r] = expf(wts[(size_t)t * top + r] - mx) / sum * scale;
    return;
  }
  const float f = renorm ? scale / (total + 1e-20f) : scale;
  for (int r = lane; r < top; r += 32) wts[(size_t)t * top + r] *= f;
}

constexpr int kMoeDownRowsPerBlock = 8;  // one output row per warp: each row already streams `top` weight rows
constexpr int kMoeRowsPerBlock = 32;  // weight rows per CTA: a decode step spreads one expert over many SMs

// hid[t, k, f] = act(W_up[ids[t,k]][f] . x[t]).  GATED 0: act = relu^2, W_up [experts, ff, width].  GATED 1: W_up [experts, 2 ff, width] with
// row 2f = gate f and row 2f + 1 = up f; hid = silu(gate . x) * (up . x).  GATED 2: the same rows, g = min(gate . x, p0), u = clamp(up . x,
// -p0, p0), hid = g * logistic(p1 * g) * (u + 1).  Grid (token, choice, slice of ff rows).
template <typename E, int GATED>
__global__ void moe_up_kernel(const E* __restrict__ xa, const E* __restrict__ w_up, const int* __restrict__ ids, E* __restrict__ hid, int width,
                              int ff, float p0, float p1) {
  extern __shared__ __align__(16) float xs[];
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int tok = blockIdx.x, k = blockIdx.y, top = gridDim.y;
  for (int i = threadIdx.x; i < width; i += blockDim.x) xs[i] = to_f(xa[(size_t)tok * width + i]);
  __syncthreads();
  const E* W = w_up + (size_t)ids[(size_t)tok * top + k] * ff * width * (GATED ? 2 : 1);
  const int f_end = min(ff, (int)(blockIdx.z + 1) * kMoeRowsPerBlock);
  for (int f = blockIdx.z * kMoeRowsPerBlock + warp; f < f_end; f += nw) {
    float r;
    if (GATED) {
      float g = warp_dot(W + (size_t)(2 * f) * width, xs, width, lane), u = warp_dot(W + (size_t)(2 * f + 1) * width, xs, width, lane);
      if (GATED == 2) {
        g = fminf(g, p0);
        u = fminf(fmaxf(u, -p0), p0);
        r = g / (1.f + expf(-p1 * g)) * (u + 1.f);
      } else {
        r = g / (1.f + expf(-g)) * u;
      }
    } else {
      const float u = fmaxf(warp_dot(W + (size_t)f * width, xs, width, lane), 0.f);
      r = u * u;
    }
    if (lane == 0) hid[((size_t)tok * top + k) * ff + f] = from_f<E>(r);
  }
}

// y[t][i] = sum_k wts[t,k] * (W_down[ids[t,k]][i] . hid[t,k]) + logistic(sg[t]) * shared[t][i]; fp32 out.  Grid (token, slice of output rows).
template <typename E>
__global__ void moe_down_kernel(const E* __restrict__ hid, const E* __restrict__ w_down, const int* __restrict__ ids, const float* __restrict__ wts,
                                const E* __restrict__ shared, const float* __restrict__ sg, float* __restrict__ y, int width, int ff, int top) {
  extern __shared__ __align__(16) float hs[];  // [top][ffp], ffp = ff rounded up to 4 so that every row starts 16-byte aligned
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int ffp = (ff + 3) & ~3;
  for (int k = 0; k < top; ++k)
    for (int f = threadIdx.x; f < ff; f += blockDim.x) hs[k * ffp + f] = to_f(hid[((size_t)t * top + k) * ff + f]);
  __syncthreads();
  const float g = shared ? (sg ? 1.f / (1.f + expf(-sg[t])) : 1.f) : 0.f;  // no gate logits: the shared expert is added as it is
  const int i_end = min(width, (int)(blockIdx.y + 1) * kMoeDownRowsPerBlock);
  for (int i = blockIdx.y * kMoeDownRowsPerBlock + warp; i < i_end; i += nw) {
    float tot = 0.f;
    for (int k = 0; k < top; ++k) {
      const E* wr = w_down + ((size_t)ids[(size_t)t * top + k] * width + i) * ff;
      tot = fmaf(wts[(size_t)t * top + k], warp_dot(wr, hs + k * ffp, ff, lane), tot);
    }
    if (lane == 0) y[(size_t)t * width + i] = tot + (shared ? g * to_f(shared[(size_t)t * width + i]) : 0.f);
  }
}

}  // namespace pk

using namespace pk;

extern "C" int pk_router_topk_ex(const float* logits, int ld, const float* correction, int* ids, float* weights, int tokens, int experts, int top,
                                int groups, int keep, float scale, int score_kind, int group_top, int renorm, pk_stream st) {
  if (!logits || !ids || !weights || tokens <= 0 || experts <= 0 || top <= 0 || groups <= 0 || experts % groups || keep <= 0 || keep > groups ||
      top > keep * (experts / groups) || ld < experts || score_kind < 0 || score_kind > 1 || group_top < 1 || group_top > 2)
    return -1;
  launch(router_grouped_topk_kernel, dim3(tokens), dim3(32), (size_t)(2 * experts + 2 * groups) * sizeof(float), st, true, logits, ld, correction, ids,
         weights, experts, top, groups, keep, scale, score_kind, group_top, renorm);
  return (int)cudaGetLastError();
}

extern "C" int pk_router_grouped_topk(const float* logits, int* ids, float* weights, int tokens, int experts, int top, int groups, int keep,
                                      float scale, pk_stream st) {
  return pk_router_topk_ex(logits, experts, nullptr, ids, weights, tokens, experts, top, groups, keep, scale, 0, 1, 1, st);
}

extern "C" int pk_moe_up_act(const void* xa, const void* w_up, const int* ids, void* hid, int tokens, int top, int width, int ff, int act, int f32,
                             pk_stream st) {
  if (act < 0 || act > 1) return -1;
  return pk_moe_up_act_p(xa, w_up, ids, hid, tokens, top, width, ff, act, 0.f, 0.f, f32, st);
}

extern "C" int pk_moe_up_act_p(const void* xa, const void* w_up, const int* ids, void* hid, int tokens, int top, int width, int ff, int act, float p0,
                               float p1, int f32, pk_stream st) {
  if (!xa || !w_up || !ids || !hid || tokens <= 0 || top <= 0 || width <= 0 || ff <= 0 || act < 0 || act > 2 || (act == 2 && !(p0 > 0.f))) return -1;
  const size_t smem = (size_t)width * sizeof(float);
  const dim3 grid(tokens, top, (ff + kMoeRowsPerBlock - 1) / kMoeRowsPerBlock);
#define PK_UP(E, G) launch(moe_up_kernel<E, G>, grid, dim3(256), smem, st, true, (const E*)xa, (const E*)w_up, ids, (E*)hid, width, ff, p0, p1)
  if (f32) {
    if (act == 2) PK_UP(float, 2);
    else if (act) PK_UP(float, 1);
    else PK_UP(float, 0);
  } else {
    if (act == 2) PK_UP(bf16, 2);
    else if (act) PK_UP(bf16, 1);
    else PK_UP(bf16, 0);
  }
#undef PK_UP
  return (int)cudaGetLastError();
}

extern "C" int pk_router_topk_logits(const float* logits, int ld, const float* bias, int* ids, float* weights, int tokens, int experts, int top,
                                     float scale, pk_stream st) {
  if (!logits || !ids || !weights || tokens <= 0 || experts <= 0 || top <= 0 || top > experts || ld < experts) return -1;
  launch(router_grouped_topk_kernel, dim3(tokens), dim3(32), (size_t)(2 * experts + 2) * sizeof(float), st, true, logits, ld, bias, ids, weights, experts,
         top, 1, 1, scale, 2, 1, 0);
  return (int)cudaGetLastError();
}

extern "C" int pk_moe_up_relu2(const void* xa, const void* w_up, const int* ids, void* hid, int tokens, int top, int width, int ff, int f32,
                               pk_stream st) {
  return pk_moe_up_act(xa, w_up, ids, hid, tokens, top, width, ff, 0, f32, st);
}

extern "C" int pk_moe_down_combine(const void* hid, const void* w_down, const int* ids, const float* weights, const void* shared,
                                   const float* shared_gate, float* y, int tokens, int top, int width, int ff, int f32, pk_stream st) {
  if (!hid || !w_down || !ids || !weights || !y || tokens <= 0 || top <= 0 || width <= 0 || ff <= 0) return -1;
  const size_t smem = (size_t)top * ((ff + 3) & ~3) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  if (f32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch(moe_down_kernel<float>, dim3(tokens, (width + kMoeDownRowsPerBlock - 1) / kMoeDownRowsPerBlock), dim3(256), smem, st, true, (const float*)hid, (const float*)w_down, ids, weights,
           (const float*)shared, shared_gate, y, width, ff, top);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch(moe_down_kernel<bf16>, dim3(tokens, (width + kMoeDownRowsPerBlock - 1) / kMoeDownRowsPerBlock), dim3(256), smem, st, true, (const bf16*)hid, (const bf16*)w_down, ids, weights, (const bf16*)shared,
           shared_gate, y, width, ff, top);
  }
  return (int)cudaGetLastError();
}
