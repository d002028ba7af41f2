// Grouped-query softmax attention over a paged K/V cache for ragged batches, with the options that newer decoder
// designs combine: projection biases, a rotary embedding over the first `dims` entries of each head from a frequency
// table (pairs interleaved (2i, 2i+1) or split in halves (i, i + dims/2); plain, YaRN or any other schedule is the
// host's table), a chunk-local causal mask (query at position p sees keys floor(p / chunk) * chunk .. p; chunk 0 = plain
// causal) and a learned per-head sink that adds exp(sink) to the softmax denominator without a value.
// Further options (pk_attn_extra): a sliding window (keys p - window + 1 .. p), a soft cap on the scaled score
// (cap * tanh(score / cap)), a linear distance bias (head h subtracts 2^(-slope_log2 (h + 1) / heads) * (p - j)), an
// element-wise logistic gate on the output, and -- in the append -- an unweighted RMS norm of every cached value head.
// A window may keep the first `keep_first` positions of the sequence visible for good (they keep their true positions).
// gqa_norm_append_kernel is the append for designs that norm q and k (per head with one weight for all heads, or over the whole
// projection at once) before rotating them, stretch the query by a factor that grows with the logarithm of the position, or
// cache the keys as projected in the place of values.
//
// Cache: token at position p of a request lives in page pages[page_off[req] + p / page_size], slot p % page_size, at
//   cache + page * page_stride + slot * (G * dim + G * vdim):  [K of G heads | V of G heads].
// Element type E (bf16 or float) for activations / cache / weights; scores, softmax and accumulation are fp32.
//   gqa_rope_append_kernel      bias + rotation of q and k, q to its buffer, k / v into the cache.  HBM-bound.
//   gqa_attention_kernel        one CTA per (query row, query head): warps stride over the visible keys with an online
//                               softmax each (lanes split the features), merged with the sink at the end.  Any sizes.
//   gqa_attention_mma_kernel    bf16 prompt portions on the tensor cores (64 query rows of one head per CTA).
#include "common.cuh"
#include "mma.cuh"
#include "typed.cuh"

namespace pk {

// qkv [tokens, ld] = [q (H*dim) | k (G*dim) | v (G*vdim)] rows of the stacked projection; bias (same layout) may be null.
template <typename E>
__global__ void gqa_rope_append_kernel(const E* __restrict__ qkv, int ld, const E* __restrict__ bias, const int* __restrict__ pos,
                                       const int* __restrict__ req, const int* __restrict__ page_off, const int* __restrict__ pages,
                                       E* __restrict__ q_out, E* __restrict__ cache, long page_stride, int page_size, int H, int G, int dim, int vdim,
                                       int dims, int interleaved, const float* __restrict__ freq, float mag, float v_eps) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x, p = pos[t];
  const E* row = qkv + (size_t)t * ld;
  const int nq = H * dim, nk = G * dim, nv = G * vdim, half = dims >> 1;
  E* slot = cache + (size_t)pages[page_off[req[t]] + p / page_size] * page_stride + (size_t)(p % page_size) * (nk + nv);
  if (v_eps > 0.f) {  // cached values are unit-RMS per head: one warp per value head
    const int lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int g = blockIdx.y * nw + (threadIdx.x >> 5); g < G; g += gridDim.y * nw) {
      const int e0 = nq + nk + g * vdim;
      float ss = 0.f;
      for (int d = lane; d < vdim; d += 32) {
        const float v = to_f(row[e0 + d]) + (bias ? to_f(bias[e0 + d]) : 0.f);
        ss = fmaf(v, v, ss);
      }
      const float inv = 1.f / sqrtf(warp_sum(ss) / (float)vdim + v_eps);
      for (int d = lane; d < vdim; d += 32) slot[e0 - nq + d] = from_f<E>((to_f(row[e0 + d]) + (bias ? to_f(bias[e0 + d]) : 0.f)) * inv);
    }
  }
  const int n_el = v_eps > 0.f ? nq + nk : nq + nk + nv;
  for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < n_el; e += gridDim.y * blockDim.x) {
    float v = to_f(row[e]) + (bias ? to_f(bias[e]) : 0.f);
    if (e < nq + nk) {
      const int d = (e < nq ? e : e - nq) % dim;
      if (d < dims) {
        int i, pe;
        bool first;
        if (interleaved) {
          i = d >> 1;
          first = (d & 1) == 0;
          pe = first ? e + 1 : e - 1;
        } else {
          first = d < half;
          i = first ? d : d - half;
          pe = first ? e + half : e - half;
        }
        const float o = to_f(row[pe]) + (bias ? to_f(bias[pe]) : 0.f);
        const float a = (float)p * freq[i];
        const float c = cosf(a) * mag, s = sinf(a) * mag;
        v = first ? v * c - o * s : v * c + o * s;
      }
    }
    if (e < nq) q_out[(size_t)t * nq + e] = from_f<E>(v);
    else slot[e - nq] = from_f<E>(v);
  }
}

// Append for designs that norm q and k before they rotate.  qkv [tokens, ld] = [q (H*dim) | k (G*dim) | v (G*vdim)]; with `v_from_k` there
// is no v part and the cached values are the keys as projected (vdim == dim).  norm_kind 1: every head of q (of k) is divided by its own
// root mean square and multiplied by qw (kw) [dim], one weight for all heads; 2: the whole q row (k row) is divided by ONE root mean
// square and multiplied by qw [H*dim] (kw [G*dim]); 0: no norm.  Then the first `dims` entries of every head rotate, and q is
// multiplied by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) (temp_every 0: not).  One CTA per token; the row lives in shared
// memory as fp32; sums of squares are added per head by one warp and then in head order, so a row's result does not depend on timing.
template <typename E>
__global__ void gqa_norm_append_kernel(const E* __restrict__ qkv, int ld, const int* __restrict__ pos, const int* __restrict__ req,
                                       const int* __restrict__ page_off, const int* __restrict__ pages, E* __restrict__ q_out, E* __restrict__ cache,
                                       long page_stride, int page_size, int H, int G, int dim, int vdim, int dims, int interleaved,
                                       const float* __restrict__ freq, float mag, const E* __restrict__ qw, const E* __restrict__ kw, int norm_kind,
                                       float eps, float temp_coef, int temp_every, int v_from_k) {
  extern __shared__ float na_sm[];
  float* row = na_sm;             // [nq + nk]
  float* inv = row + (H + G) * dim;  // [H + G] sum of squares per head
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x, p = pos[t], lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const E* src = qkv + (size_t)t * ld;
  const int nq = H * dim, nk = G * dim, nv = G * vdim, half = dims >> 1;
  // the page lookup (three dependent loads) and the weights of the last phase travel while the row is loaded and summed
  const int page = pages[page_off[req[t]] + p / page_size];
  if (norm_kind)
    for (int e = threadIdx.x * 64; e < (norm_kind == 1 ? dim : nq + nk); e += blockDim.x * 64)
      prefetch_l2(norm_kind == 1 ? (e < dim ? qw + e : kw + e - dim) : (e < nq ? qw + e : kw + e - nq));  // a line of 64 entries each
  if (norm_kind == 1 && threadIdx.x * 64 < dim) prefetch_l2(kw + threadIdx.x * 64);
  // 16-byte accesses where every piece of the row and of the slot starts on such a boundary (bf16, sizes multiples of 8)
  const bool vec = sizeof(E) == 2 && ((nq | nk | nv | ld | (int)(page_stride & 7)) & 7) == 0 &&
                   ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(cache)) & 15) == 0;
  if (vec) {
    for (int e = threadIdx.x * 8; e < nq + nk; e += blockDim.x * 8) {
      const uint4 u = *reinterpret_cast<const uint4*>(src + e);
      *reinterpret_cast<float4*>(row + e) = make_float4(bf16_lo(u.x), bf16_hi(u.x), bf16_lo(u.y), bf16_hi(u.y));
      *reinterpret_cast<float4*>(row + e + 4) = make_float4(bf16_lo(u.z), bf16_hi(u.z), bf16_lo(u.w), bf16_hi(u.w));
    }
  } else {
    for (int e = threadIdx.x; e < nq + nk; e += blockDim.x) row[e] = to_f(src[e]);
  }
  __syncthreads();
  if (norm_kind) {
    for (int hd = warp; hd < H + G; hd += nw) {
      float ss = 0.f;
      for (int d = lane; d < dim; d += 32) ss = fmaf(row[hd * dim + d], row[hd * dim + d], ss);
      ss = warp_sum(ss);
      if (lane == 0) inv[hd] = ss;
    }
    __syncthreads();
  }
  // reciprocal root mean square of the whole q row / k row (norm_kind 2): the heads' sums added in head order by every thread
  float iq = 1.f, ik = 1.f;
  if (norm_kind == 2) {
    float sq = 0.f, sk = 0.f;
    for (int hd = 0; hd < H; ++hd) sq += inv[hd];
    for (int hd = 0; hd < G; ++hd) sk += inv[H + hd];
    iq = 1.f / sqrtf(sq / (float)nq + eps);
    ik = 1.f / sqrtf(sk / (float)nk + eps);
  }
  const float stretch = temp_every > 0 ? 1.f + temp_coef * logf((float)((p + 1) / temp_every) + 1.f) : 1.f;
  E* slot = cache + (size_t)page * page_stride + (size_t)(p % page_size) * (nk + nv);
  // norm, rotation and the query's factor head by head (a warp per head, lanes over its entries: no index arithmetic per entry)
  for (int hd = warp; hd < H + G; hd += nw) {
    const bool is_q = hd < H;
    const float f = norm_kind == 1 ? 1.f / sqrtf(inv[hd] / (float)dim + eps) : norm_kind == 2 ? (is_q ? iq : ik) : 1.f;
    const E* w = norm_kind == 1 ? (is_q ? qw : kw) : norm_kind == 2 ? (is_q ? qw + hd * dim : kw + (hd - H) * dim) : nullptr;
    const float* hrow = row + hd * dim;
    E* dst = is_q ? q_out + (size_t)t * nq + hd * dim : slot + (hd - H) * dim;
    const float out_f = is_q ? stretch : 1.f;
    for (int d = lane; d < dim; d += 32) {
      float v = hrow[d] * f * (w ? to_f(w[d]) : 1.f);
      if (d < dims) {
        int i, pd;
        bool first;
        if (interleaved) {
          i = d >> 1;
          first = (d & 1) == 0;
          pd = first ? d + 1 : d - 1;
        } else {
          first = d < half;
          i = first ? d : d - half;
          pd = first ? d + half : d - half;
        }
        const float o = hrow[pd] * f * (w ? to_f(w[pd]) : 1.f);
        const float a = (float)p * freq[i];
        const float c = cosf(a) * mag, sn = sinf(a) * mag;
        v = first ? v * c - o * sn : v * c + o * sn;
      }
      dst[d] = from_f<E>(v * out_f);
    }
  }
  const E* vsrc = src + (v_from_k ? nq : nq + nk);  // the values: the keys as projected, or the value projection
  const int n_val = v_from_k ? nk : nv;
  if (vec) {
    for (int e = threadIdx.x * 8; e < n_val; e += blockDim.x * 8) *reinterpret_cast<uint4*>(slot + nk + e) = *reinterpret_cast<const uint4*>(vsrc + e);
  } else {
    for (int e = threadIdx.x; e < n_val; e += blockDim.x) slot[nk + e] = vsrc[e];
  }
}

// the options of pk_attn_extra as the kernels take them (all off when zero / null)
struct AttnExtra {
  int window;
  float softcap, slope_log2;
  const void* gate;
  long gate_ld;
  int max_kv_len;
  int keep_first;
};
__device__ __forceinline__ int first_visible(int p, int chunk, int window) {
  int lo = chunk > 0 ? (p / chunk) * chunk : 0;
  if (window > 0) lo = max(lo, p - window + 1);
  return lo;
}
__device__ __forceinline__ float head_slope(float slope_log2, int h, int H) { return slope_log2 > 0.f ? exp2f(-slope_log2 * (float)(h + 1) / (float)H) : 0.f; }
// scaled score -> soft cap -> minus the distance bias
__device__ __forceinline__ float shape_score(float s, float softcap, float slope, int distance) {
  if (softcap > 0.f) s = softcap * tanhf(s / softcap);
  return s - slope * (float)distance;
}
// 2^x on the special-function unit (relative error about 2^-22; 2^-inf = 0)
__device__ __forceinline__ float fast_ex2(float v) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;

constexpr int kGqaWarps = 8;
constexpr int kGqaMaxPerLane = 8;  // features per lane: dim, vdim <= 256

template <typename E>
__global__ void __launch_bounds__(kGqaWarps * 32) gqa_attention_kernel(const E* __restrict__ q, const E* __restrict__ cache, const E* __restrict__ sink,
                                                                      const int* __restrict__ pos, const int* __restrict__ req,
                                                                      const int* __restrict__ page_off, const int* __restrict__ pages,
                                                                      E* __restrict__ out, long page_stride, int page_size, int H, int G, int dim,
                                                                      int vdim, float scale, int chunk, AttnExtra x) {
  __shared__ float sm_m[kGqaWarps], sm_l[kGqaWarps];
  extern __shared__ float sm_acc[];  // [warps][vdim]
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x, h = blockIdx.y, g = h / (H / G), lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int p = pos[t], lo = first_visible(p, chunk, x.window);
  const float slope = head_slope(x.slope_log2, h, H);
  const int* pg = pages + page_off[req[t]];
  const int tok = G * (dim + vdim);
  float qr[kGqaMaxPerLane], acc[kGqaMaxPerLane];
#pragma unroll
  for (int i = 0; i < kGqaMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    qr[i] = d < dim ? to_f(q[((size_t)t * H + h) * dim + d]) * scale : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  // visible keys: the first `nf` positions (kept for good, when the window has left them behind), then lo .. p
  const int nf = min(x.keep_first, lo), n_vis = nf + p - lo + 1;
  // two keys per trip (i and i + warps): their loads, dot products and exponentials overlap, which halves the dependent chain per key
  for (int i = warp; i < n_vis; i += 2 * kGqaWarps) {
    const int i2 = i + kGqaWarps;
    const bool two = i2 < n_vis;
    const int j = i < nf ? i : lo + (i - nf), j2 = i2 < nf ? i2 : lo + (i2 - nf);
    const E* kv_a = cache + (size_t)pg[j / page_size] * page_stride + (size_t)(j % page_size) * tok;
    const E* kv_b = two ? cache + (size_t)pg[j2 / page_size] * page_stride + (size_t)(j2 % page_size) * tok : kv_a;
    float ka[kGqaMaxPerLane], kb[kGqaMaxPerLane], va[kGqaMaxPerLane], vb[kGqaMaxPerLane];
#pragma unroll
    for (int i = 0; i < kGqaMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      ka[i] = d < dim ? to_f(kv_a[g * dim + d]) : 0.f;
      kb[i] = d < dim ? to_f(kv_b[g * dim + d]) : 0.f;
      va[i] = d < vdim ? to_f(kv_a[G * dim + g * vdim + d]) : 0.f;
      vb[i] = d < vdim ? to_f(kv_b[G * dim + g * vdim + d]) : 0.f;
    }
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int i = 0; i < kGqaMaxPerLane; ++i) {
      sa = fmaf(qr[i], ka[i], sa);
      sb = fmaf(qr[i], kb[i], sb);
    }
    sa = shape_score(warp_sum(sa), x.softcap, slope, p - j);
    sb = two ? shape_score(warp_sum(sb), x.softcap, slope, p - j2) : -INFINITY;
    const float mn = fmaxf(m, fmaxf(sa, sb)), c = expf(m - mn), ea = expf(sa - mn), eb = two ? expf(sb - mn) : 0.f;
    l = l * c + (ea + eb);
#pragma unroll
    for (int i = 0; i < kGqaMaxPerLane; ++i) acc[i] = acc[i] * c + (ea * va[i] + eb * vb[i]);
    m = mn;
  }
  if (lane == 0) {
    sm_m[warp] = m;
    sm_l[warp] = l;
  }
#pragma unroll
  for (int i = 0; i < kGqaMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < vdim) sm_acc[warp * vdim + d] = acc[i];
  }
  __syncthreads();
  const float sk = sink ? to_f(sink[h]) : -INFINITY;
  float mt = sk;
#pragma unroll
  for (int w = 0; w < kGqaWarps; ++w) mt = fmaxf(mt, sm_m[w]);
  float den = sink ? expf(sk - mt) : 0.f;
  float cw[kGqaWarps];
#pragma unroll
  for (int w = 0; w < kGqaWarps; ++w) {
    cw[w] = sm_m[w] == -INFINITY ? 0.f : expf(sm_m[w] - mt);
    den += sm_l[w] * cw[w];
  }
  for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < kGqaWarps; ++w) o += sm_acc[w * vdim + d] * cw[w];
    o /= den;
    if (x.gate) o *= 1.f / (1.f + expf(-to_f(static_cast<const E*>(x.gate)[(size_t)t * x.gate_ld + h * vdim + d])));
    out[((size_t)t * H + h) * vdim + d] = from_f<E>(o);
  }
}

// ---- tensor cores (bf16): one CTA = 64 consecutive rows of the step (4 warps x 16 rows) for one query head.  Rows of a
// tile may belong to several requests: the tile walks each request's visible key range in 64-key blocks with the other
// rows masked.  dim, vdim multiples of 16 up to 128.  K and V blocks go through a two-stage cp.async ring in shared memory (the
// next block's copy overlaps this block's products); S = Q K^T and O += P V with mma.sync m16n8k16, P rounded to bf16 for the
// second product, statistics in fp32.
constexpr int kAmRows = 64, kAmKeys = 64;

template <int DQ, int DV>
__global__ void __launch_bounds__(128, 3) gqa_attention_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ cache, const bf16* __restrict__ sink,
                                                               const int* __restrict__ pos, const int* __restrict__ req,
                                                               const int* __restrict__ page_off, const int* __restrict__ pages,
                                                               bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                                                               long page_stride, int page_size, int T, int H, int G, float scale, int chunk,
                                                               AttnExtra x) {
  constexpr int LDK = DQ + 8, LDV = DV + 8;
  extern __shared__ __align__(16) unsigned char am_smem[];  // two stages of [keys][LDK] K and [keys][LDV] V
  bf16* const Ks0 = reinterpret_cast<bf16*>(am_smem);
  bf16* const Vs0 = Ks0 + 2 * kAmKeys * LDK;
  __shared__ int s_req[kAmRows], s_pos[kAmRows];
  __shared__ long long s_slot[2][kAmKeys];  // per stage: element offset of every key row's cache slot (-1: not to be read)
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  // grid (head, tile, split): the heads of a tile start together (a group's heads read the same keys), and the tiles run from the
  // end of the step backwards, so that the CTAs that start last are the ones with the fewest visible keys
  const int t0 = (gridDim.y - 1 - blockIdx.y) * kAmRows, h = blockIdx.x, g = h / (H / G);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gq = lane >> 2, tq = lane & 3;
  if (tid < kAmRows) {
    const int t = t0 + tid;
    s_req[tid] = t < T ? req[t] : -1;
    s_pos[tid] = t < T ? pos[t] : -1;
  }
  __syncthreads();
  const int tok = G * (DQ + DV);
  // this warp's rows: r0 = warp * 16 + gq and r0 + 8
  const int ra = warp * 16 + gq, rb = ra + 8;
  const int req_a = s_req[ra], req_b = s_req[rb], pos_a = s_pos[ra], pos_b = s_pos[rb];
  const int lo_a = pos_a >= 0 ? first_visible(pos_a, chunk, x.window) : 0, lo_b = pos_b >= 0 ? first_visible(pos_b, chunk, x.window) : 0;
  // The tensor-core kernel keeps scores in units of log2 (every exponential is one ex2), and shapes a raw score q.k with
  //   cap * tanh(z) = cap - 2 cap / (e^(2z) + 1),  z = q.k * scale / cap      (fast exponential and reciprocal: absolute error of a few
  //   1e-7 of the cap, far below the bf16 rounding of P)
  const bool capped = x.softcap > 0.f;
  const float slope2 = head_slope(x.slope_log2, h, H) * kLog2e, cap2 = x.softcap * kLog2e;
  const float c1 = capped ? 2.f * scale / x.softcap * kLog2e : scale * kLog2e;  // raw score -> ex2 argument of e^(2z) / -> plain scaled score
  const int split = blockIdx.z, nsplit = gridDim.z;  // few rows: every request's 64-key blocks are dealt out to gridDim.z CTAs
  // Q fragments (A operand, row-major 16 x DQ)
  uint32_t qa[DQ / 16][4];
#pragma unroll
  for (int kk = 0; kk < DQ / 16; ++kk) {
    const int c = kk * 16 + 2 * tq;
    const bf16* qra = q + ((size_t)(t0 + ra) * H + h) * DQ + c;
    const bf16* qrb = q + ((size_t)(t0 + rb) * H + h) * DQ + c;
    qa[kk][0] = req_a >= 0 ? *reinterpret_cast<const uint32_t*>(qra) : 0u;
    qa[kk][1] = req_b >= 0 ? *reinterpret_cast<const uint32_t*>(qrb) : 0u;
    qa[kk][2] = req_a >= 0 ? *reinterpret_cast<const uint32_t*>(qra + 8) : 0u;
    qa[kk][3] = req_b >= 0 ? *reinterpret_cast<const uint32_t*>(qrb + 8) : 0u;
  }
  float oa[DV / 8][4] = {};
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  // requests of the tile are contiguous runs: walk them one after the other
  int r_first = 0;
  while (r_first < kAmRows && s_req[r_first] >= 0) {
    const int rq = s_req[r_first];
    int r_last = r_first;
    while (r_last + 1 < kAmRows && s_req[r_last + 1] == rq) ++r_last;
    const int p_min = s_pos[r_first], p_max = s_pos[r_last];
    const int k_lo = first_visible(p_min, chunk, x.window);
    const int* pg = pages + page_off[rq];
    // stage `buf` <- keys k0 .. k0 + 63 of this request (cp.async; rows outside [k_lo, p_max] and not among the kept first are zero-filled)
    auto load = [&](int k0, int buf) {
      bf16* Kd = Ks0 + buf * kAmKeys * LDK;
      bf16* Vd = Vs0 + buf * kAmKeys * LDV;
      if (tid < kAmKeys) {  // one page-table read per key row, not one per 16-byte piece
        const int j = k0 + tid;
        s_slot[buf][tid] = (j <= p_max && (j >= k_lo || j < x.keep_first)) ? (long long)pg[j / page_size] * page_stride + (long long)(j % page_size) * tok : -1;
      }
      __syncthreads();
#pragma unroll 4
      for (int c = tid; c < kAmKeys * (DQ / 8); c += 128) {
        const int r = c / (DQ / 8), cc = (c % (DQ / 8)) * 8;
        const long long at = s_slot[buf][r];
        if (at >= 0) cp_async16(&Kd[r * LDK + cc], cache + at + g * DQ + cc);
        else *reinterpret_cast<uint4*>(&Kd[r * LDK + cc]) = make_uint4(0, 0, 0, 0);
      }
#pragma unroll 4
      for (int c = tid; c < kAmKeys * (DV / 8); c += 128) {
        const int r = c / (DV / 8), cc = (c % (DV / 8)) * 8;
        const long long at = s_slot[buf][r];
        if (at >= 0) cp_async16(&Vd[r * LDV + cc], cache + at + G * DQ + g * DV + cc);
        else *reinterpret_cast<uint4*>(&Vd[r * LDV + cc]) = make_uint4(0, 0, 0, 0);
      }
      cp_async_commit();
    };
    // blocks to walk: those that hold kept first keys and lie wholly before the window's first block, then the window's blocks
    const int k_start = k_lo - (k_lo % kAmKeys);
    const int n_kept = min((x.keep_first + kAmKeys - 1) / kAmKeys, k_start / kAmKeys);
    const int n_blocks = n_kept + (p_max - k_start) / kAmKeys + 1, per_split = (n_blocks + nsplit - 1) / nsplit;
    const int b_first = split * per_split, b_end = min(n_blocks, b_first + per_split);
    auto block_k0 = [&](int b) { return b < n_kept ? b * kAmKeys : k_start + (b - n_kept) * kAmKeys; };
    __syncthreads();  // the previous request's readers are done with both stages
    if (b_first < b_end) load(block_k0(b_first), 0);
    for (int b = b_first, it = 0; b < b_end; ++b, ++it) {
      const int buf = it & 1, k0 = block_k0(b);
      cp_async_wait_all();
      __syncthreads();  // this block has landed, and nobody reads the other stage any more
      if (b + 1 < b_end) load(block_k0(b + 1), buf ^ 1);  // overlaps the products below
      const bf16* Ks = Ks0 + buf * kAmKeys * LDK;
      const bf16* Vs = Vs0 + buf * kAmKeys * LDV;
      const bool on_a = req_a == rq, on_b = req_b == rq;
      if (!__any_sync(0xffffffffu, on_a || on_b)) continue;  // warp-uniform: the tensor-core instructions below need all 32 lanes
      // S = Q K^T: 16 rows x 64 keys per warp
      float s[kAmKeys / 8][4] = {};
#pragma unroll
      for (int kk = 0; kk < DQ / 16; ++kk)
#pragma unroll
        for (int np = 0; np < kAmKeys / 16; ++np) {
          uint32_t b[4];
          ldsm_x4(b, &Ks[(np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * LDK + kk * 16 + ((lane >> 3) & 1) * 8]);
          mma_bf16_16816(s[np * 2], qa[kk], b[0], b[1]);
          mma_bf16_16816(s[np * 2 + 1], qa[kk], b[2], b[3]);
        }
      // key j = k0 + 2 tq + c of this thread's column c is seen from a row at position p iff 0 <= p - j <= p - first_visible(p)
      const int da = on_a ? pos_a - k0 - 2 * tq : -(1 << 20), db = on_b ? pos_b - k0 - 2 * tq : -(1 << 20);
      const unsigned span_a = on_a ? pos_a - lo_a : 0, span_b = on_b ? pos_b - lo_b : 0;
      const float fa = (float)da, fb = (float)db;
      const int kept = x.keep_first - k0 - 2 * tq;  // column c holds one of the kept first keys iff c < kept
      float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
      for (int ni = 0; ni < kAmKeys / 8; ++ni)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int c = ni * 8 + (e & 1);
          const bool top = e < 2;
          const int dist = (top ? da : db) - c;
          const bool ok = (unsigned)dist <= (top ? span_a : span_b) || (c < kept && dist >= 0);
          float v = s[ni][e] * c1;
          if (capped) v = fmaf(-2.f * cap2, __fdividef(1.f, fast_ex2(fminf(v, 80.f)) + 1.f), cap2);
          v = fmaf(-slope2, (top ? fa : fb) - (float)c, v);
          v = ok ? v : -INFINITY;
          s[ni][e] = v;
          if (top) mx_a = fmaxf(mx_a, v);
          else mx_b = fmaxf(mx_b, v);
        }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
      // a row that has seen nothing yet keeps its maximum at -inf; subtracting 0 instead leaves its (all -inf) scores at 2^-inf = 0
      const float sub_a = mn_a == -INFINITY ? 0.f : mn_a, sub_b = mn_b == -INFINITY ? 0.f : mn_b;
      const float c_a = fast_ex2(m_a - sub_a), c_b = fast_ex2(m_b - sub_b);
      float sum_a = 0.f, sum_b = 0.f;
      uint32_t pa[kAmKeys / 16][4];
#pragma unroll
      for (int ni = 0; ni < kAmKeys / 8; ++ni) {
        // P is rounded to bf16 once, for the second product; the row sum adds the rounded values
        const uint32_t pk_a = pack_bf16(fast_ex2(s[ni][0] - sub_a), fast_ex2(s[ni][1] - sub_a));
        const uint32_t pk_b = pack_bf16(fast_ex2(s[ni][2] - sub_b), fast_ex2(s[ni][3] - sub_b));
        sum_a += bf16_lo(pk_a) + bf16_hi(pk_a);
        sum_b += bf16_lo(pk_b) + bf16_hi(pk_b);
        pa[ni >> 1][(ni & 1) * 2] = pk_a;
        pa[ni >> 1][(ni & 1) * 2 + 1] = pk_b;
      }
      sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
      sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
      sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
      sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
      l_a = l_a * c_a + sum_a;
      l_b = l_b * c_b + sum_b;
      m_a = mn_a;
      m_b = mn_b;
#pragma unroll
      for (int ni = 0; ni < DV / 8; ++ni) {
        oa[ni][0] *= c_a;
        oa[ni][1] *= c_a;
        oa[ni][2] *= c_b;
        oa[ni][3] *= c_b;
      }
      // O += P V: V block is [keys][DV] row-major = the B operand's k-major form through ldmatrix.trans
#pragma unroll
      for (int kk = 0; kk < kAmKeys / 16; ++kk)
#pragma unroll
        for (int np = 0; np < DV / 16; ++np) {
          uint32_t b[4];
          ldsm_x4_trans(b, &Vs[(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + np * 16 + ((lane >> 4) & 1) * 8]);
          mma_bf16_16816(oa[np * 2], pa[kk], b[0], b[1]);
          mma_bf16_16816(oa[np * 2 + 1], pa[kk], b[2], b[3]);
        }
    }
    r_first = r_last + 1;
  }
  if (nsplit > 1) {  // partial state (running maximum, sum, unnormalised output) of this split; gqa_attention_merge_kernel finishes the rows
    const size_t sa = ((size_t)(h * nsplit + split) * T + (t0 + ra)), sb = ((size_t)(h * nsplit + split) * T + (t0 + rb));
    if (req_a >= 0 && tq == 0) part_ml[sa * 2] = m_a * kLn2, part_ml[sa * 2 + 1] = l_a;  // maxima leave in natural units
    if (req_b >= 0 && tq == 0) part_ml[sb * 2] = m_b * kLn2, part_ml[sb * 2 + 1] = l_b;
#pragma unroll
    for (int ni = 0; ni < DV / 8; ++ni) {
      const int c = ni * 8 + 2 * tq;
      if (req_a >= 0) *reinterpret_cast<float2*>(part_o + sa * DV + c) = make_float2(oa[ni][0], oa[ni][1]);
      if (req_b >= 0) *reinterpret_cast<float2*>(part_o + sb * DV + c) = make_float2(oa[ni][2], oa[ni][3]);
    }
    return;
  }
  const float sk = sink ? bf2f(sink[h]) * kLog2e : -INFINITY;  // the sink joins in the same log2 units
  const float mt_a = fmaxf(m_a, sk), mt_b = fmaxf(m_b, sk);
  const float f_a = m_a == -INFINITY ? 0.f : exp2f(m_a - mt_a), f_b = m_b == -INFINITY ? 0.f : exp2f(m_b - mt_b);
  const float d_a = l_a * f_a + (sink ? exp2f(sk - mt_a) : 0.f), d_b = l_b * f_b + (sink ? exp2f(sk - mt_b) : 0.f);
  const float i_a = f_a / d_a, i_b = f_b / d_b;
#pragma unroll
  for (int ni = 0; ni < DV / 8; ++ni) {
    const int c = ni * 8 + 2 * tq;
    float g0 = 1.f, g1 = 1.f, g2 = 1.f, g3 = 1.f;
    if (x.gate) {
      const bf16* ga = static_cast<const bf16*>(x.gate) + (size_t)(t0 + ra) * x.gate_ld + h * DV + c;
      const bf16* gb = static_cast<const bf16*>(x.gate) + (size_t)(t0 + rb) * x.gate_ld + h * DV + c;
      if (req_a >= 0) g0 = 1.f / (1.f + expf(-bf2f(ga[0]))), g1 = 1.f / (1.f + expf(-bf2f(ga[1])));
      if (req_b >= 0) g2 = 1.f / (1.f + expf(-bf2f(gb[0]))), g3 = 1.f / (1.f + expf(-bf2f(gb[1])));
    }
    if (req_a >= 0) *reinterpret_cast<uint32_t*>(out + ((size_t)(t0 + ra) * H + h) * DV + c) = pack_bf16(oa[ni][0] * i_a * g0, oa[ni][1] * i_a * g1);
    if (req_b >= 0) *reinterpret_cast<uint32_t*>(out + ((size_t)(t0 + rb) * H + h) * DV + c) = pack_bf16(oa[ni][2] * i_b * g2, oa[ni][3] * i_b * g3);
  }
}

// one CTA per (row, head): combine the splits' (m, l, O), join the sink, apply the output gate
__global__ void gqa_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const bf16* __restrict__ sink,
                                           bf16* __restrict__ out, int nsplit, int T, int H, int vdim, AttnExtra x) {
  __shared__ float wgt[64];  // per split: exp(m_s - M) / denominator
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x, h = blockIdx.y;
  if (threadIdx.x < 32) {
    const float sk = sink ? bf2f(sink[h]) : -INFINITY;
    float m[2], l[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int sp = threadIdx.x + 32 * i;
      const size_t slot = (size_t)(h * nsplit + sp) * T + t;
      m[i] = sp < nsplit ? part_ml[slot * 2] : -INFINITY;
      l[i] = sp < nsplit ? part_ml[slot * 2 + 1] : 0.f;
    }
    const float M = fmaxf(warp_max(fmaxf(m[0], m[1])), sk);  // finite: a query always sees its own position
    const float e0 = m[0] == -INFINITY ? 0.f : expf(m[0] - M), e1 = m[1] == -INFINITY ? 0.f : expf(m[1] - M);
    const float inv = 1.f / (warp_sum(l[0] * e0 + l[1] * e1) + (sink ? expf(sk - M) : 0.f));
    wgt[threadIdx.x] = e0 * inv;
    wgt[threadIdx.x + 32] = e1 * inv;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
    float a4[4] = {0.f, 0.f, 0.f, 0.f};
    int sp = 0;
    for (; sp + 4 <= nsplit; sp += 4) {  // the splits' loads are independent: four in flight
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = part_o[((size_t)(h * nsplit + sp + u) * T + t) * vdim + d];
#pragma unroll
      for (int u = 0; u < 4; ++u) a4[u] = fmaf(v[u], wgt[sp + u], a4[u]);
    }
    for (; sp < nsplit; ++sp) a4[0] = fmaf(part_o[((size_t)(h * nsplit + sp) * T + t) * vdim + d], wgt[sp], a4[0]);
    float o = (a4[0] + a4[1]) + (a4[2] + a4[3]);
    if (x.gate) o *= 1.f / (1.f + expf(-bf2f(static_cast<const bf16*>(x.gate)[(size_t)t * x.gate_ld + h * vdim + d])));
    out[((size_t)t * H + h) * vdim + d] = f2bf(o);
  }
}

template <int DQ, int DV>
static void launch_gqa_mma(const bf16* q, const bf16* cache, const bf16* sink, const int* pos, const int* req, const int* page_off, const int* pages,
                           bf16* out, long page_stride, int page_size, int T, int H, int G, float scale, int chunk, AttnExtra x, cudaStream_t st) {
  const size_t smem = (size_t)2 * kAmKeys * (DQ + 8 + DV + 8) * sizeof(bf16);
  static bool attr_set = false;  // per template instance
  if (!attr_set) {
    cudaFuncSetAttribute(gqa_attention_mma_kernel<DQ, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr_set = true;
  }
  // Few rows (decode steps): the key axis is dealt out to several CTAs per (tile, head) so that the step fills the GPU.  The span a
  // row can see is bounded by the window / chunk, else by the longest context of the step (when the caller knows it).
  const int tiles = (T + kAmRows - 1) / kAmRows;
  int span = x.max_kv_len;
  if (x.window > 0) span = span > 0 ? min(span, x.window + x.keep_first + T) : x.window + x.keep_first + T;
  if (chunk > 0) span = span > 0 ? min(span, chunk) : chunk;
  int splits = 1;
  ThreadState& ts = tls();
  if (T < kAmRows && span > 2 * kAmKeys && ts.scratch) {
    const int blocks = (span + kAmKeys - 1) / kAmKeys + 1;
    splits = min(min(blocks, (2 * sm_count() + tiles * H - 1) / (tiles * H)), 64);
    while (splits > 1 && (size_t)H * splits * T * (DV + 2) * sizeof(float) > ts.scratch_bytes) --splits;
  }
  float* po = static_cast<float*>(ts.scratch);
  float* pml = po ? po + (size_t)H * splits * T * DV : nullptr;
  launch(gqa_attention_mma_kernel<DQ, DV>, dim3(H, tiles, splits), dim3(128), smem, st, true, q, cache, sink, pos, req, page_off, pages, out, po, pml,
         page_stride, page_size, T, H, G, scale, chunk, x);
  if (splits > 1)
    launch(gqa_attention_merge_kernel, dim3(T, H), dim3(DV >= 128 ? 128 : 64), 0, st, true, (const float*)po, (const float*)pml, sink, out, splits, T, H, DV, x);
}

}  // namespace pk

using namespace pk;

extern "C" int pk_gqa_rope_append(const void* qkv, int ld, const void* bias, const int* positions, const int* req, const int* page_off,
                                  const int* pages, void* q_out, void* cache, long page_stride, int page_size, int heads, int kv_heads, int dim,
                                  int vdim, int dims, int interleaved, const float* freq, float mag, int tokens, int f32, pk_stream st) {
  return pk_gqa_rope_append_ex(qkv, ld, bias, positions, req, page_off, pages, q_out, cache, page_stride, page_size, heads, kv_heads, dim, vdim, dims,
                               interleaved, freq, mag, 0.f, tokens, f32, st);
}

extern "C" int pk_gqa_rope_append_ex(const void* qkv, int ld, const void* bias, const int* positions, const int* req, const int* page_off,
                                     const int* pages, void* q_out, void* cache, long page_stride, int page_size, int heads, int kv_heads, int dim,
                                     int vdim, int dims, int interleaved, const float* freq, float mag, float value_norm_eps, int tokens, int f32,
                                     pk_stream st) {
  if (!qkv || !positions || !req || !page_off || !pages || !q_out || !cache || tokens <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads ||
      dim <= 0 || vdim <= 0 || dims < 0 || dims > dim || (dims & 1) || (dims > 0 && !freq) || page_size <= 0)
    return -1;
  // few tokens (decoding): a token's features are spread over several CTAs
  const int n_all = heads * dim + kv_heads * (dim + vdim);
  const dim3 grid(tokens, tokens >= 128 ? 1 : std::min((n_all + 255) / 256, 16));
  if (f32)
    launch(gqa_rope_append_kernel<float>, grid, dim3(256), 0, st, true, (const float*)qkv, ld, (const float*)bias, positions, req, page_off, pages,
           (float*)q_out, (float*)cache, page_stride, page_size, heads, kv_heads, dim, vdim, dims, interleaved, freq, mag, value_norm_eps);
  else
    launch(gqa_rope_append_kernel<bf16>, grid, dim3(256), 0, st, true, (const bf16*)qkv, ld, (const bf16*)bias, positions, req, page_off, pages,
           (bf16*)q_out, (bf16*)cache, page_stride, page_size, heads, kv_heads, dim, vdim, dims, interleaved, freq, mag, value_norm_eps);
  return (int)cudaGetLastError();
}

extern "C" int pk_gqa_norm_append(const void* qkv, int ld, const int* positions, const int* req, const int* page_off, const int* pages, void* q_out,
                                  void* cache, long page_stride, int page_size, int heads, int kv_heads, int dim, int vdim, int dims, int interleaved,
                                  const float* freq, float mag, const pk_qk_prep* prep, int tokens, int f32, pk_stream st) {
  if (!qkv || !positions || !req || !page_off || !pages || !q_out || !cache || !prep || tokens <= 0 || heads <= 0 || kv_heads <= 0 ||
      heads % kv_heads || dim <= 0 || vdim <= 0 || dims < 0 || dims > dim || (dims & 1) || (dims > 0 && !freq) || page_size <= 0 ||
      prep->norm_kind < 0 || prep->norm_kind > 2 || (prep->norm_kind && (!prep->q_weight || !prep->k_weight)) || prep->temp_every < 0 ||
      (prep->values_are_keys && vdim != dim))
    return -1;
  const size_t smem = ((size_t)(heads + kv_heads) * dim + heads + kv_heads) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  const int threads = tokens > 64 ? 256 : std::min(1024, std::max(128, ((heads + kv_heads) * dim / 2 + 31) / 32 * 32));
#define PK_NA(E)                                                                                                                                   \
  do {                                                                                                                                             \
    if (smem > 48 * 1024) cudaFuncSetAttribute(gqa_norm_append_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);                \
    launch(gqa_norm_append_kernel<E>, dim3(tokens), dim3(threads), smem, st, true, (const E*)qkv, ld, positions, req, page_off, pages, (E*)q_out,  \
           (E*)cache, page_stride, page_size, heads, kv_heads, dim, vdim, dims, interleaved, freq, mag, (const E*)prep->q_weight,                  \
           (const E*)prep->k_weight, prep->norm_kind, prep->eps, prep->temp_coef, prep->temp_every, prep->values_are_keys);                        \
  } while (0)
  if (f32) PK_NA(float);
  else PK_NA(bf16);
#undef PK_NA
  return (int)cudaGetLastError();
}

extern "C" int pk_gqa_attention(const void* q, const void* cache, const void* sink, const int* positions, const int* req, const int* page_off,
                                const int* pages, void* out, long page_stride, int page_size, int tokens, int heads, int kv_heads, int dim,
                                int vdim, float scale, int chunk, int f32, pk_stream st) {
  return pk_gqa_attention_ex(q, cache, sink, positions, req, page_off, pages, out, page_stride, page_size, tokens, heads, kv_heads, dim, vdim, scale,
                             chunk, nullptr, f32, st);
}

extern "C" int pk_gqa_attention_ex(const void* q, const void* cache, const void* sink, const int* positions, const int* req, const int* page_off,
                                   const int* pages, void* out, long page_stride, int page_size, int tokens, int heads, int kv_heads, int dim,
                                   int vdim, float scale, int chunk, const pk_attn_extra* extra, int f32, pk_stream st) {
  if (!q || !cache || !positions || !req || !page_off || !pages || !out || tokens <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads ||
      dim <= 0 || vdim <= 0 || chunk < 0 || page_size <= 0)
    return -1;
  AttnExtra x{0, 0.f, 0.f, nullptr, 0, 0, 0};
  if (extra) {
    if (extra->window < 0 || extra->softcap < 0.f || extra->slope_log2 < 0.f || extra->max_kv_len < 0 || extra->keep_first < 0) return -1;
    x = AttnExtra{extra->window, extra->softcap, extra->slope_log2, extra->gate, extra->gate_ld, extra->max_kv_len, extra->window > 0 ? extra->keep_first : 0};
  }
  if (dim > 32 * kGqaMaxPerLane || vdim > 32 * kGqaMaxPerLane) return -2;
  const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
                       page_stride % 8 == 0;
  // bf16 prompt portions always; single decoded tokens too when the caller asked through the _ex entry (the key axis is then split)
  if (!f32 && (tokens >= 32 || extra) && aligned && dim == vdim && (dim == 64 || dim == 128 || dim == 32 || dim == 96) && (dim * kv_heads) % 8 == 0) {
#define PK_GQA_MMA(D) \
  launch_gqa_mma<D, D>((const bf16*)q, (const bf16*)cache, (const bf16*)sink, positions, req, page_off, pages, (bf16*)out, page_stride, page_size, tokens, heads, kv_heads, scale, chunk, x, st)
    if (dim == 32) PK_GQA_MMA(32);
    else if (dim == 64) PK_GQA_MMA(64);
    else if (dim == 96) PK_GQA_MMA(96);
    else PK_GQA_MMA(128);
#undef PK_GQA_MMA
    return (int)cudaGetLastError();
  }
  const size_t smem = (size_t)kGqaWarps * vdim * sizeof(float);
  if (f32)
    launch(gqa_attention_kernel<float>, dim3(tokens, heads), dim3(kGqaWarps * 32), smem, st, true, (const float*)q, (const float*)cache, (const float*)sink,
           positions, req, page_off, pages, (float*)out, page_stride, page_size, heads, kv_heads, dim, vdim, scale, chunk, x);
  else
    launch(gqa_attention_kernel<bf16>, dim3(tokens, heads), dim3(kGqaWarps * 32), smem, st, true, (const bf16*)q, (const bf16*)cache, (const bf16*)sink,
           positions, req, page_off, pages, (bf16*)out, page_stride, page_size, heads, kv_heads, dim, vdim, scale, chunk, x);
  return (int)cudaGetLastError();
}
