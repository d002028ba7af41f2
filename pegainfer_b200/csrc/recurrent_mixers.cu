// Recurrent mixers with a matrix state per head, for ragged batches whose requests keep their state in numbered slots:
//   * short causal convolution + SiLU over time per channel, with the last taps - 1 inputs of every request as state;
//   * gated delta rule:   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q        (q, k unit vectors per head)
//   * xLSTM matrix memory: m' = max(f + m, i);  S <- e^(f + m - m') S + e^(i - m') k v^T;  n likewise with k alone;
//                          o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)        (i, f soft-capped log gates, m starts at 0)
//     slot layout: S [H][dim][vdim], n [H][dim], m [H][vdim + 1] (every column keeps its own copy of the running maximum)
//   * state-space duality (scalar decay per head):  S <- e^(-e^(A_log) dt) S + dt B x^T;  y = S^T C + D x,  dt = softplus(. + dt_bias)
//     (B, C of the head's group [state], x the head's slice [vdim]; the state S [state][vdim] takes the place of [dim][vdim])
//   * per-head RMS norm of the read-out times a weight times an activation of a gate projection (or the gate first, then the norm).
// State, gates, decays, unit norms and the recurrences are fp32 whatever the element type E of the activations is.
//
// Step layout: entry e of the step owns rows [row0[e], row0[e] + len[e]) of every [tokens, features] buffer (a portion
// of a prompt or one decoded token) and the state slot slot[e]; a slot's state is `state + slot * slot_stride` floats.
// Sequence kernels: one CTA per (entry, head, slice of value columns); a column of S lives in the registers of DK / 16
// neighbouring lanes (key size padded to the template's DK), tokens run one after the other; per block of 32 tokens all
// threads first bring q, k, v and the gate inputs into shared memory and turn them into unit vectors / gates.  The matrix
// memory's normaliser n is one more column with value 1.  Latency-bound per token (48 FMAs and two shuffle reductions per
// thread, one warp per scheduler).
#include "common.cuh"
#include "typed.cuh"

namespace pk {

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float logsigmoidf_(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// y[t][c] = silu(bias[c] + sum_j w[c][j] * x[t - (taps-1-j)][c]) (bias may be null); inputs before this step's rows come from the slot's state
// [taps-1][C] (oldest first; zero for a new request).  in / out may have different row strides; out may alias nothing of in.
template <typename E>
__global__ void causal_conv_silu_kernel(const E* __restrict__ in, int ld_in, const E* __restrict__ w, const E* __restrict__ bias, const float* __restrict__ state, long slot_stride,
                                        const int* __restrict__ req, const int* __restrict__ slot, const int* __restrict__ row0, E* __restrict__ out,
                                        int ld_out, int C, int taps, long total) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int t = (int)(i / C), c = (int)(i % C), e = req[t], off = t - row0[e];
    const float* st = state + (size_t)slot[e] * slot_stride;
    float acc = bias ? to_f(bias[c]) : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;
      const float x = off - back >= 0 ? to_f(in[(size_t)(t - back) * ld_in + c]) : st[(size_t)(taps - 1 + off - back) * C + c];
      acc = fmaf(to_f(w[(size_t)c * taps + j]), x, acc);
    }
    out[(size_t)t * ld_out + c] = from_f<E>(acc / (1.f + expf(-acc)));
  }
}

// after the step: the slot keeps the last taps - 1 inputs (old ones move up when the portion was shorter)
template <typename E>
__global__ void conv_state_update_kernel(const E* __restrict__ in, int ld_in, float* __restrict__ state, long slot_stride, const int* __restrict__ slot,
                                         const int* __restrict__ row0, const int* __restrict__ len, int C, int taps) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int e = blockIdx.y, n = len[e], r0 = row0[e];
  float* st = state + (size_t)slot[e] * slot_stride;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < C; c += gridDim.x * blockDim.x)
    for (int s = 0; s < taps - 1; ++s) {
      const int o = n - (taps - 1) + s;
      st[(size_t)s * C + c] = o >= 0 ? to_f(in[(size_t)(r0 + o) * ld_in + c]) : st[(size_t)(s + n) * C + c];
    }
}

struct SeqArgs {
  const void* qkv;     // [tokens, ld]: q at q_off + kv_head * dim, k at k_off + kv_head * dim, v at v_off + head * vdim
  int ld, q_off, k_off, v_off;
  const float* z;      // [tokens, ldz] fp32 few-row projections: z[za_off + head], z[zb_off + head]
  int ldz, za_off, zb_off;
  const float* p0;     // delta: A_log [H];  matrix memory: input-gate bias [H]
  const float* p1;     // delta: dt_bias [H];  matrix memory: forget-gate bias [H]
  float* state;        // slot base (this layer's block)
  long slot_stride;
  const int *slot, *row0, *len;
  float* out;          // [tokens, H * vdim] fp32 read-out
  float* den;          // matrix memory: [tokens, H] divisor
  int H, G, dim, vdim;
  float cap;           // matrix memory: gate soft cap
  const void* dt;      // state space: [tokens, ld_dt] element type, step-size projection of head h at dt_off + h
  int ld_dt, dt_off;
  const float* p2;     // state space: skip weight D [H]  (p0 = A_log, p1 = dt_bias)
};

// MODE 0: gated delta rule.  MODE 1: xLSTM matrix memory.  MODE 2: state-space duality (q = C, k = B, v = x; dim = state size).
// Thread layout: KS = DK / 16 neighbouring lanes share one state column, each holding 16 of its DK entries in registers
// (entry (m * KS + ks) * 4 + e for m < 4, e < 4, so that the lanes' 16-byte reads of k / q from shared memory fall on
// consecutive banks); the two dot products per token are finished with log2(KS) shuffles.  128 / KS columns per CTA; the
// matrix memory's normaliser column rides in one more warp of the head's first CTA.
template <typename E, int DK, int MODE>
__global__ void __launch_bounds__(160) recurrent_seq_kernel(SeqArgs a) {
  constexpr int KS = DK / 16, COLS = 128 / KS, TB = DK <= 128 ? 32 : 16, NS = 16;  // NS state entries per thread
  __shared__ __align__(16) float ks[TB][DK];
  __shared__ __align__(16) float qs[TB][DK];
  __shared__ float vs[TB][COLS];
  __shared__ float g0[TB], g1[TB];  // delta: decay, write strength;  memory: log forget gate, log input gate
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int e = blockIdx.x, h = blockIdx.y, kvh = h / (a.H / a.G);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  const int n = a.len[e], r0 = a.row0[e], dim = a.dim, vdim = a.vdim;
  const int cl = tid / KS, ksi = tid % KS;  // column inside the CTA, share of the key axis
  const int col0 = blockIdx.z * COLS, col = col0 + cl;
  const bool is_v = tid < 128 && col < vdim;
  const bool is_n = MODE == 1 && blockIdx.z == 0 && tid >= 128 && tid < 128 + KS;
  float* base = a.state + (size_t)a.slot[e] * a.slot_stride;
  float* S_g = base + (size_t)h * dim * vdim;                      // [dim][vdim]
  float* n_g = base + (size_t)a.H * dim * vdim + (size_t)h * dim;  // matrix memory only
  // one copy of the running maximum per column: CTAs of a head never read what another one wrote
  float* m_g = base + (size_t)a.H * dim * vdim + (size_t)a.H * dim + (size_t)h * (vdim + 1) + (is_v ? col : vdim);
  float S[NS];
#pragma unroll
  for (int j = 0; j < NS; ++j) {
    const int i = ((j >> 2) * KS + ksi) * 4 + (j & 3);
    S[j] = i < dim ? (is_v ? S_g[(size_t)i * vdim + col] : (is_n ? n_g[i] : 0.f)) : 0.f;
  }
  float m = (MODE == 1 && (is_v || is_n)) ? m_g[0] : 0.f;
  const E* X = static_cast<const E*>(a.qkv);
  const float qscale = 1.f / sqrtf((float)dim);
  const size_t out_ld = (size_t)a.H * vdim;
  for (int b0 = 0; b0 < n; b0 += TB) {
    const int nb = min(TB, n - b0);
    __syncthreads();  // the previous block's readers are done
    // 1. raw q, k, v and gate inputs of the block's tokens (independent loads, many in flight)
    const E* Xb = X + (size_t)(r0 + b0) * a.ld;
    bool staged = false;
    if constexpr (sizeof(E) == 2) {
      // 16-byte pieces of 8 bf16 when every row slice starts on a 16-byte boundary
      const int qo = a.q_off + kvh * dim, ko = a.k_off + kvh * dim, vo = a.v_off + h * vdim + col0;
      if (((a.ld | qo | ko | vo | dim | vdim) & 7) == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0) {
        staged = true;
        constexpr int PR = DK / 8;
        for (int i = tid; i < nb * PR; i += blockDim.x) {
          const int tt = i / PR, d0 = (i % PR) * 8;
          const E* row = Xb + (size_t)tt * a.ld;
          uint4 qv = make_uint4(0, 0, 0, 0), kv = qv;
          if (d0 < dim) {
            qv = *reinterpret_cast<const uint4*>(row + qo + d0);
            kv = *reinterpret_cast<const uint4*>(row + ko + d0);
          }
          *reinterpret_cast<float4*>(&qs[tt][d0]) = make_float4(bf16_lo(qv.x), bf16_hi(qv.x), bf16_lo(qv.y), bf16_hi(qv.y));
          *reinterpret_cast<float4*>(&qs[tt][d0 + 4]) = make_float4(bf16_lo(qv.z), bf16_hi(qv.z), bf16_lo(qv.w), bf16_hi(qv.w));
          *reinterpret_cast<float4*>(&ks[tt][d0]) = make_float4(bf16_lo(kv.x), bf16_hi(kv.x), bf16_lo(kv.y), bf16_hi(kv.y));
          *reinterpret_cast<float4*>(&ks[tt][d0 + 4]) = make_float4(bf16_lo(kv.z), bf16_hi(kv.z), bf16_lo(kv.w), bf16_hi(kv.w));
        }
        constexpr int PV = COLS / 8;
        for (int i = tid; i < nb * PV; i += blockDim.x) {
          const int tt = i / PV, c0 = (i % PV) * 8;
          uint4 vv = make_uint4(0, 0, 0, 0);
          if (col0 + c0 < vdim) vv = *reinterpret_cast<const uint4*>(Xb + (size_t)tt * a.ld + vo + c0);
          vs[tt][c0] = bf16_lo(vv.x), vs[tt][c0 + 1] = bf16_hi(vv.x), vs[tt][c0 + 2] = bf16_lo(vv.y), vs[tt][c0 + 3] = bf16_hi(vv.y);
          vs[tt][c0 + 4] = bf16_lo(vv.z), vs[tt][c0 + 5] = bf16_hi(vv.z), vs[tt][c0 + 6] = bf16_lo(vv.w), vs[tt][c0 + 7] = bf16_hi(vv.w);
        }
      }
    }
#pragma unroll 4
    for (int i = staged ? nb * DK : tid; i < nb * DK; i += blockDim.x) {
      const int tt = i / DK, d = i % DK;
      const E* row = Xb + (size_t)tt * a.ld;
      qs[tt][d] = d < dim ? to_f(row[a.q_off + kvh * dim + d]) : 0.f;
      ks[tt][d] = d < dim ? to_f(row[a.k_off + kvh * dim + d]) : 0.f;
    }
#pragma unroll 4
    for (int i = staged ? nb * COLS : tid; i < nb * COLS; i += blockDim.x) {
      const int tt = i / COLS, c = i % COLS;
      vs[tt][c] = col0 + c < vdim ? to_f(Xb[(size_t)tt * a.ld + a.v_off + h * vdim + col0 + c]) : 0.f;
    }
    if (MODE == 2) {
      if (tid < nb) {  // step size and decay of the head at this token, from the projection's output
        const float step = softplusf_(to_f(static_cast<const E*>(a.dt)[(size_t)(r0 + b0 + tid) * a.ld_dt + a.dt_off + h]) + a.p1[h]);
        g0[tid] = expf(-expf(a.p0[h]) * step);
        g1[tid] = step;
      }
    } else if (tid < nb) {
      const size_t row = (size_t)(r0 + b0 + tid);
      const float za = a.z[row * a.ldz + a.za_off + h], zb = a.z[row * a.ldz + a.zb_off + h];
      if (MODE == 0) {  // za: decay projection, zb: write-strength projection
        g0[tid] = expf(-expf(a.p0[h]) * softplusf_(za + a.p1[h]));
        g1[tid] = sigmoidf_(zb);
      } else {  // za: forget gate, zb: input gate
        g0[tid] = logsigmoidf_(a.cap * tanhf((za + a.p1[h]) / a.cap));
        g1[tid] = a.cap * tanhf((zb + a.p0[h]) / a.cap);
      }
    }
    __syncthreads();
    // 2. unit vectors (delta rule) and the query's scale
    for (int tt = warp; MODE != 2 && tt < nb; tt += nw) {
      float qf = qscale, kf = 1.f;
      if (MODE == 0) {
        float qq = 0.f, kk = 0.f;
        for (int i = lane; i < DK; i += 32) {
          qq = fmaf(qs[tt][i], qs[tt][i], qq);
          kk = fmaf(ks[tt][i], ks[tt][i], kk);
        }
        qq = warp_sum(qq);
        kk = warp_sum(kk);
        qf = qscale / sqrtf(qq + 1e-6f);
        kf = 1.f / sqrtf(kk + 1e-6f);
      }
      for (int i = lane; i < DK; i += 32) {
        qs[tt][i] *= qf;
        if (MODE == 0) ks[tt][i] *= kf;
      }
    }
    __syncthreads();
    if (warp >= 4 && !(MODE == 1 && blockIdx.z == 0)) continue;  // the extra warp only carries the normaliser
    // 3. the recurrence, token by token (whole warps run it: the shuffles below need every lane)
#pragma unroll 2
    for (int tt = 0; tt < nb; ++tt) {
      const size_t row = (size_t)(r0 + b0 + tt);
      const float vt = tid < 128 ? vs[tt][cl] : 1.f;
      const float4* k4p = reinterpret_cast<const float4*>(&ks[tt][0]) + ksi;
      const float4* q4p = reinterpret_cast<const float4*>(&qs[tt][0]) + ksi;
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
      if (MODE == 0) {
        const float g = g0[tt], beta = g1[tt];
        float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
#pragma unroll
        for (int mi = 0; mi < NS / 4; ++mi) {
          const float4 k4 = k4p[mi * KS];
          S[mi * 4] *= g;
          S[mi * 4 + 1] *= g;
          S[mi * 4 + 2] *= g;
          S[mi * 4 + 3] *= g;
          c0 = fmaf(S[mi * 4], k4.x, c0);
          c1 = fmaf(S[mi * 4 + 1], k4.y, c1);
          c2 = fmaf(S[mi * 4 + 2], k4.z, c2);
          c3 = fmaf(S[mi * 4 + 3], k4.w, c3);
        }
        float kv = (c0 + c1) + (c2 + c3);
#pragma unroll
        for (int o = 1; o < KS; o <<= 1) kv += __shfl_xor_sync(0xffffffffu, kv, o);
        const float u = beta * (vt - kv);
#pragma unroll
        for (int mi = 0; mi < NS / 4; ++mi) {
          const float4 k4 = k4p[mi * KS];
          const float4 q4 = q4p[mi * KS];
          S[mi * 4] = fmaf(k4.x, u, S[mi * 4]);
          S[mi * 4 + 1] = fmaf(k4.y, u, S[mi * 4 + 1]);
          S[mi * 4 + 2] = fmaf(k4.z, u, S[mi * 4 + 2]);
          S[mi * 4 + 3] = fmaf(k4.w, u, S[mi * 4 + 3]);
          o0 = fmaf(S[mi * 4], q4.x, o0);
          o1 = fmaf(S[mi * 4 + 1], q4.y, o1);
          o2 = fmaf(S[mi * 4 + 2], q4.z, o2);
          o3 = fmaf(S[mi * 4 + 3], q4.w, o3);
        }
        float o = (o0 + o1) + (o2 + o3);
#pragma unroll
        for (int s = 1; s < KS; s <<= 1) o += __shfl_xor_sync(0xffffffffu, o, s);
        if (is_v && ksi == 0) a.out[row * out_ld + h * vdim + col] = o;
      } else if (MODE == 2) {
        const float fa = g0[tt], wb = g1[tt] * vt;
#pragma unroll
        for (int mi = 0; mi < NS / 4; ++mi) {
          const float4 k4 = k4p[mi * KS];
          const float4 q4 = q4p[mi * KS];
          S[mi * 4] = fmaf(k4.x, wb, fa * S[mi * 4]);
          S[mi * 4 + 1] = fmaf(k4.y, wb, fa * S[mi * 4 + 1]);
          S[mi * 4 + 2] = fmaf(k4.z, wb, fa * S[mi * 4 + 2]);
          S[mi * 4 + 3] = fmaf(k4.w, wb, fa * S[mi * 4 + 3]);
          o0 = fmaf(S[mi * 4], q4.x, o0);
          o1 = fmaf(S[mi * 4 + 1], q4.y, o1);
          o2 = fmaf(S[mi * 4 + 2], q4.z, o2);
          o3 = fmaf(S[mi * 4 + 3], q4.w, o3);
        }
        float o = (o0 + o1) + (o2 + o3);
#pragma unroll
        for (int s = 1; s < KS; s <<= 1) o += __shfl_xor_sync(0xffffffffu, o, s);
        if (is_v && ksi == 0) a.out[row * out_ld + h * vdim + col] = fmaf(a.p2[h], vt, o);
      } else {
        const float f = g0[tt], ig = g1[tt];
        const float mn = fmaxf(f + m, ig);
        const float fa = expf(f + m - mn), wb = expf(ig - mn) * vt;
        m = mn;
#pragma unroll
        for (int mi = 0; mi < NS / 4; ++mi) {
          const float4 k4 = k4p[mi * KS];
          const float4 q4 = q4p[mi * KS];
          S[mi * 4] = fmaf(k4.x, wb, fa * S[mi * 4]);
          S[mi * 4 + 1] = fmaf(k4.y, wb, fa * S[mi * 4 + 1]);
          S[mi * 4 + 2] = fmaf(k4.z, wb, fa * S[mi * 4 + 2]);
          S[mi * 4 + 3] = fmaf(k4.w, wb, fa * S[mi * 4 + 3]);
          o0 = fmaf(S[mi * 4], q4.x, o0);
          o1 = fmaf(S[mi * 4 + 1], q4.y, o1);
          o2 = fmaf(S[mi * 4 + 2], q4.z, o2);
          o3 = fmaf(S[mi * 4 + 3], q4.w, o3);
        }
        float o = (o0 + o1) + (o2 + o3);
#pragma unroll
        for (int s = 1; s < KS; s <<= 1) o += __shfl_xor_sync(0xffffffffu, o, s);
        if (is_v && ksi == 0) a.out[row * out_ld + h * vdim + col] = o;
        else if (is_n && ksi == 0) a.den[row * a.H + h] = fmaxf(fabsf(o), expf(-mn)) + 1e-6f;
      }
    }
  }
  if (is_v || is_n) {
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      const int i = ((j >> 2) * KS + ksi) * 4 + (j & 3);
      if (i < dim) {
        if (is_v) S_g[(size_t)i * vdim + col] = S[j];
        else n_g[i] = S[j];
      }
    }
    if (MODE == 1 && ksi == 0) m_g[0] = m;
  }
}

// out[t, h, j] = E( (o[t,h,j] / den[t,h]) / sqrt(mean_j(.^2) + eps) * w[h * w_stride + j] * act(gate[t, gate_off + h*vdim + j]) )
// act 0: silu, 1: logistic.  act 2: the silu gate comes BEFORE the norm, out = rms_norm(o * silu(gate)) * w.  den may be null.
// One warp per (token, head); "head" may be any equal part of the row (norm groups).
template <typename E>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ den, const E* __restrict__ w, int w_stride,
                                      const E* __restrict__ gate, int ld_gate, int gate_off, E* __restrict__ out, int H, int vdim, float eps, int act,
                                      long pairs) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int lane = threadIdx.x & 31;
  const long pr = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pr >= pairs) return;
  const long t = pr / H;
  const int h = (int)(pr % H);
  const float* orow = o + pr * vdim;
  float ss = 0.f;
  for (int j = lane; j < vdim; j += 32) {
    float v = den ? orow[j] / den[pr] : orow[j];
    if (act == 2) {
      const float gz = to_f(gate[(size_t)t * ld_gate + gate_off + h * vdim + j]);
      v *= gz / (1.f + expf(-gz));
    }
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)vdim + eps);
  for (int j = lane; j < vdim; j += 32) {
    const float v = den ? orow[j] / den[pr] : orow[j];
    const float gz = to_f(gate[(size_t)t * ld_gate + gate_off + h * vdim + j]);
    const float ga = act == 1 ? 1.f / (1.f + expf(-gz)) : gz / (1.f + expf(-gz));
    out[pr * vdim + j] = from_f<E>(act == 2 ? (v * ga) * inv * to_f(w[(size_t)h * w_stride + j]) : v * inv * to_f(w[(size_t)h * w_stride + j]) * ga);
  }
}

// the same for few (token, head) pairs of many entries each (a decode step with wide norm groups): one CTA per pair
template <typename E>
__global__ void head_norm_gate_wide_kernel(const float* __restrict__ o, const float* __restrict__ den, const E* __restrict__ w, int w_stride,
                                           const E* __restrict__ gate, int ld_gate, int gate_off, E* __restrict__ out, int H, int vdim, float eps,
                                           int act) {
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const long pr = blockIdx.x, t = pr / H;
  const int h = (int)(pr % H);
  const float* orow = o + pr * vdim;
  const float dn = den ? den[pr] : 1.f;
  float v[4], ga[4];  // up to 4 entries per thread (vdim <= 4 * blockDim.x)
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int j = threadIdx.x + u * blockDim.x;
    v[u] = 0.f;
    ga[u] = 0.f;
    if (j < vdim) {
      const float gz = to_f(gate[(size_t)t * ld_gate + gate_off + h * vdim + j]);
      ga[u] = act == 1 ? 1.f / (1.f + expf(-gz)) : gz / (1.f + expf(-gz));
      v[u] = den ? orow[j] / dn : orow[j];
      if (act == 2) v[u] *= ga[u];
      ss = fmaf(v[u], v[u], ss);
    }
  }
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)vdim + eps);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int j = threadIdx.x + u * blockDim.x;
    if (j < vdim) out[pr * vdim + j] = from_f<E>(act == 2 ? v[u] * inv * to_f(w[(size_t)h * w_stride + j]) : v[u] * inv * to_f(w[(size_t)h * w_stride + j]) * ga[u]);
  }
}

template <typename E, int MODE>
static int launch_seq(const SeqArgs& a, int entries, cudaStream_t st) {
  if (a.dim > 256) return -2;
  const int dk = a.dim <= 32 ? 32 : a.dim <= 64 ? 64 : a.dim <= 128 ? 128 : 256;
  const int cols = 128 / (dk / 16);
  const dim3 grid(entries, a.H, (a.vdim + cols - 1) / cols), block(MODE == 1 ? 160 : 128);
  if (dk == 32) launch(recurrent_seq_kernel<E, 32, MODE>, grid, block, 0, st, true, a);
  else if (dk == 64) launch(recurrent_seq_kernel<E, 64, MODE>, grid, block, 0, st, true, a);
  else if (dk == 128) launch(recurrent_seq_kernel<E, 128, MODE>, grid, block, 0, st, true, a);
  else launch(recurrent_seq_kernel<E, 256, MODE>, grid, block, 0, st, true, a);
  return (int)cudaGetLastError();
}

static inline int grid_for(long n, int block) { return (int)std::min<long>((n + block - 1) / block, 148L * 16); }

}  // namespace pk

using namespace pk;

extern "C" int pk_causal_conv_silu(const void* in, int ld_in, const void* w, float* state, long slot_stride, const int* req, const int* slot,
                                   const int* row0, const int* len, void* out, int ld_out, int channels, int taps, int tokens, int entries, int f32,
                                   pk_stream st) {
  return pk_causal_conv_silu_bias(in, ld_in, w, nullptr, state, slot_stride, req, slot, row0, len, out, ld_out, channels, taps, tokens, entries, f32, st);
}

extern "C" int pk_causal_conv_silu_bias(const void* in, int ld_in, const void* w, const void* bias, float* state, long slot_stride, const int* req,
                                        const int* slot, const int* row0, const int* len, void* out, int ld_out, int channels, int taps, int tokens,
                                        int entries, int f32, pk_stream st) {
  if (!in || !w || !state || !req || !slot || !row0 || !len || !out || channels <= 0 || taps <= 0 || tokens <= 0 || entries <= 0) return -1;
  const long total = (long)tokens * channels;
  if (f32)
    launch(causal_conv_silu_kernel<float>, dim3(grid_for(total, 256)), dim3(256), 0, st, true, (const float*)in, ld_in, (const float*)w, (const float*)bias,
           (const float*)state, slot_stride, req, slot, row0, (float*)out, ld_out, channels, taps, total);
  else
    launch(causal_conv_silu_kernel<bf16>, dim3(grid_for(total, 256)), dim3(256), 0, st, true, (const bf16*)in, ld_in, (const bf16*)w, (const bf16*)bias,
           (const float*)state, slot_stride, req, slot, row0, (bf16*)out, ld_out, channels, taps, total);
  if (taps > 1) {
    const dim3 g((channels + 255) / 256, entries);
    if (f32) launch(conv_state_update_kernel<float>, g, dim3(256), 0, st, true, (const float*)in, ld_in, state, slot_stride, slot, row0, len, channels, taps);
    else launch(conv_state_update_kernel<bf16>, g, dim3(256), 0, st, true, (const bf16*)in, ld_in, state, slot_stride, slot, row0, len, channels, taps);
  }
  return (int)cudaGetLastError();
}

static bool seq_args_ok(const void* qkv, const float* z, const float* p0, const float* p1, float* state, const int* slot, const int* row0, const int* len,
                        float* out, int H, int G, int dim, int vdim, int entries) {
  return qkv && z && p0 && p1 && state && slot && row0 && len && out && H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && entries > 0;
}

extern "C" int pk_gated_delta_seq(const void* qkv, int ld, int q_off, int k_off, int v_off, const float* z, int ldz, int decay_off, int beta_off,
                                  const float* a_log, const float* dt_bias, float* state, long slot_stride, const int* slot, const int* row0,
                                  const int* len, float* out, int heads, int kv_heads, int dim, int vdim, int entries, int f32, pk_stream st) {
  if (!seq_args_ok(qkv, z, a_log, dt_bias, state, slot, row0, len, out, heads, kv_heads, dim, vdim, entries)) return -1;
  SeqArgs a{qkv, ld, q_off, k_off, v_off, z, ldz, decay_off, beta_off, a_log, dt_bias, state, slot_stride, slot, row0, len, out, nullptr,
            heads, kv_heads, dim, vdim, 0.f};
  return f32 ? launch_seq<float, 0>(a, entries, st) : launch_seq<bf16, 0>(a, entries, st);
}

extern "C" int pk_mlstm_seq(const void* qkv, int ld, int q_off, int k_off, int v_off, const float* z, int ldz, int forget_off, int input_off,
                            const float* input_bias, const float* forget_bias, float cap, float* state, long slot_stride, const int* slot,
                            const int* row0, const int* len, float* out, float* den, int heads, int dim, int vdim, int entries, int f32,
                            pk_stream st) {
  if (!seq_args_ok(qkv, z, input_bias, forget_bias, state, slot, row0, len, out, heads, heads, dim, vdim, entries) || !den || !(cap > 0.f)) return -1;
  SeqArgs a{qkv, ld, q_off, k_off, v_off, z, ldz, forget_off, input_off, input_bias, forget_bias, state, slot_stride, slot, row0, len, out, den,
            heads, heads, dim, vdim, cap};
  return f32 ? launch_seq<float, 1>(a, entries, st) : launch_seq<bf16, 1>(a, entries, st);
}

extern "C" int pk_head_norm_gate(const float* o, const float* den, const void* w, int w_stride, const void* gate, int ld_gate, int gate_off, void* out,
                                 int tokens, int heads, int vdim, float eps, int act, int f32, pk_stream st) {
  if (!o || !w || !gate || !out || tokens <= 0 || heads <= 0 || vdim <= 0 || act < 0 || act > 2) return -1;
  const long pairs = (long)tokens * heads;
  if (vdim >= 256 && vdim <= 4096 && pairs <= 1024) {  // few wide pairs: a CTA each, so that a decode step is not one warp's loop
    const dim3 gw((unsigned)pairs), bw(vdim <= 512 ? 128 : vdim <= 1024 ? 256 : 1024);
    if (f32)
      launch(head_norm_gate_wide_kernel<float>, gw, bw, 0, st, true, o, den, (const float*)w, w_stride, (const float*)gate, ld_gate, gate_off, (float*)out,
             heads, vdim, eps, act);
    else
      launch(head_norm_gate_wide_kernel<bf16>, gw, bw, 0, st, true, o, den, (const bf16*)w, w_stride, (const bf16*)gate, ld_gate, gate_off, (bf16*)out,
             heads, vdim, eps, act);
    return (int)cudaGetLastError();
  }
  const dim3 g((unsigned)((pairs + 3) / 4));
  if (f32)
    launch(head_norm_gate_kernel<float>, g, dim3(128), 0, st, true, o, den, (const float*)w, w_stride, (const float*)gate, ld_gate, gate_off, (float*)out,
           heads, vdim, eps, act, pairs);
  else
    launch(head_norm_gate_kernel<bf16>, g, dim3(128), 0, st, true, o, den, (const bf16*)w, w_stride, (const bf16*)gate, ld_gate, gate_off, (bf16*)out, heads,
           vdim, eps, act, pairs);
  return (int)cudaGetLastError();
}

extern "C" int pk_ssd_seq(const void* xbc, int ld, int x_off, int b_off, int c_off, const void* dt, int ld_dt, int dt_off, const float* a_log,
                          const float* dt_bias, const float* d_skip, float* state, long slot_stride, const int* slot, const int* row0, const int* len,
                          float* out, int heads, int groups, int state_dim, int vdim, int entries, int f32, pk_stream st) {
  if (!xbc || !dt || !a_log || !dt_bias || !d_skip || !state || !slot || !row0 || !len || !out || heads <= 0 || groups <= 0 || heads % groups ||
      state_dim <= 0 || vdim <= 0 || entries <= 0)
    return -1;
  SeqArgs a{xbc, ld, c_off, b_off, x_off, nullptr, 0, 0, 0, a_log, dt_bias, state, slot_stride, slot, row0, len, out, nullptr,
            heads, groups, state_dim, vdim, 0.f, dt, ld_dt, dt_off, d_skip};
  return f32 ? launch_seq<float, 2>(a, entries, st) : launch_seq<bf16, 2>(a, entries, st);
}
