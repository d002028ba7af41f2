// Ops for models that keep an fp32 residual stream and norm the OUTPUT of a sublayer (x <- x + norm(f(x))):
// embedding into fp32, RMS norm with a weight stored as an offset from one fused with the residual add and the cast that
// feeds the next projection, final norm over gathered rows, a skinny fp32 projection (routers, gates), activations, and
// a strided batched GEMM in plain FMA arithmetic (true fp32 when the element type is float; per-head factor products of
// the latent attention in either type).  Every kernel is templated on the activation / weight element type E
// (bf16 or float); arithmetic is fp32 throughout and a value is rounded once, when it is stored as E.
// All of these are HBM-bound except the GEMM: 4 - 12 bytes per element per pass.
#include <algorithm>

#include "common.cuh"
#include "typed.cuh"

namespace pk {

template <typename E>
__global__ void embed_res32_kernel(const E* __restrict__ embed, const int* __restrict__ tok, float* __restrict__ x,
                                   E* __restrict__ xa, int width) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x;
  const E* row = embed + (size_t)tok[t] * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const E v = row[i];
    x[(size_t)t * width + i] = to_f(v);
    xa[(size_t)t * width + i] = v;
  }
}

// x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * (1 + w);  xa[t] = E(x[t]).  Y is E or float.
template <typename E, typename Y>
__global__ void offset_norm_residual_kernel(const Y* __restrict__ y, const E* __restrict__ w, float* __restrict__ x,
                                            E* __restrict__ xa, int width, float eps) {
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x;
  const Y* yr = y + (size_t)t * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = to_f(yr[i]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float r = x[(size_t)t * width + i] + to_f(yr[i]) * inv * (1.f + to_f(w[i]));
    x[(size_t)t * width + i] = r;
    xa[(size_t)t * width + i] = from_f<E>(r);
  }
}

// out[r] = E(x[rows[r]] / rms * (1 + w)): the model's last norm, only for the rows whose logits are wanted
template <typename E>
__global__ void offset_norm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, const E* __restrict__ w,
                                        E* __restrict__ out, int width, float eps) {
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const float* xr = x + (size_t)rows[blockIdx.x] * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) ss += xr[i] * xr[i];
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    out[(size_t)blockIdx.x * width + i] = from_f<E>(xr[i] * inv * (1.f + to_f(w[i])));
}

// out[t][m] = sum_k W[m][k] x[t][k] with the fp32 residual as input: one warp per output
template <typename E>
__global__ void skinny_proj_kernel(const E* __restrict__ W, const float* __restrict__ x, float* __restrict__ out, int M, int K) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const float* xr = x + (size_t)t * K;
  for (int m = blockIdx.y * nw + warp; m < M; m += gridDim.y * nw) {
    const float acc = warp_dot(W + (size_t)m * K, xr, K, lane);
    if (lane == 0) out[(size_t)t * M + m] = acc;
  }
}

// kind 0: out[t][f] = silu(in[t][f]) * in[t][F + f]   (in is [T, 2F]: gate rows stacked over up rows)
// kind 1: out[t][f] = relu(in[t][f])^2                (in is [T, F])
template <typename E>
__global__ void act_kernel(const E* __restrict__ in, E* __restrict__ out, int F, long total, int kind) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long t = i / F, f = i % F;
    float r;
    if (kind == 0) {
      const float g = to_f(in[t * 2 * F + f]), u = to_f(in[t * 2 * F + F + f]);
      r = g / (1.f + expf(-g)) * u;
    } else {
      const float u = fmaxf(to_f(in[i]), 0.f);
      r = u * u;
    }
    out[i] = from_f<E>(r);
  }
}

template <typename A, typename B>
__global__ void convert_kernel(const A* __restrict__ in, B* __restrict__ out, long n) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) out[i] = from_f<B>(to_f(in[i]));
}

// C[b][i][j] = (sum_k A[b*bsA + i*lda + k] * B[b*bsB + k*sbk + j*sbn]) * f(row_scale[i*ld_scale + b])
// f = identity (scale_kind 1) or logistic (scale_kind 2); no scale when row_scale is null.  64 x 64 output tile, 256 threads, 4 x 4 each.
template <typename E>
__global__ void gemm_strided_kernel(const E* __restrict__ A, const E* __restrict__ B, E* __restrict__ C, const float* __restrict__ row_scale,
                                    int rows, int cols, int K, long lda, long sbk, long sbn, long ldc, long bsA, long bsB, long bsC,
                                    int ld_scale, int scale_kind) {
  constexpr int TL = 64, KT = 16;
  __shared__ float as[KT][TL + 1], bs[KT][TL + 1];
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int b = blockIdx.z;
  A += (size_t)b * bsA;
  B += (size_t)b * bsB;
  C += (size_t)b * bsC;
  const int i0 = blockIdx.y * TL, j0 = blockIdx.x * TL;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += KT) {
    for (int e = threadIdx.x; e < TL * KT; e += 256) {
      const int r = e / KT, c = e % KT;  // consecutive threads walk k: contiguous for A (and for B when sbk == 1)
      as[c][r] = (i0 + r < rows && k0 + c < K) ? to_f(A[(size_t)(i0 + r) * lda + k0 + c]) : 0.f;
    }
    if (sbk == 1) {
      for (int e = threadIdx.x; e < TL * KT; e += 256) {
        const int r = e / KT, c = e % KT;
        bs[c][r] = (j0 + r < cols && k0 + c < K) ? to_f(B[(size_t)(j0 + r) * sbn + k0 + c]) : 0.f;
      }
    } else {
      for (int e = threadIdx.x; e < TL * KT; e += 256) {
        const int c = e / TL, r = e % TL;  // consecutive threads walk j
        bs[c][r] = (j0 + r < cols && k0 + c < K) ? to_f(B[(size_t)(k0 + c) * sbk + (size_t)(j0 + r) * sbn]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < KT; ++c) {
      float av[4], bv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        av[u] = as[c][ty * 4 + u];
        bv[u] = bs[c][tx * 4 + u];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < 4; ++v) acc[u][v] = fmaf(av[u], bv[v], acc[u][v]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i = i0 + ty * 4 + u;
    if (i >= rows) continue;
    float s = 1.f;
    if (row_scale) {
      s = row_scale[(size_t)i * ld_scale + b];
      if (scale_kind == 2) s = 1.f / (1.f + expf(-s));
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int j = j0 + tx * 4 + v;
      if (j < cols) C[(size_t)i * ldc + j] = from_f<E>(acc[u][v] * s);
    }
  }
}

// The same product for a few rows (decode) when B is K-contiguous (sbk == 1): grid (row, batch, slice of columns); the A row
// is staged as fp32 in shared memory and every warp streams whole B rows.
template <typename E>
__global__ void gemm_strided_rows_kernel(const E* __restrict__ A, const E* __restrict__ B, E* __restrict__ C, const float* __restrict__ row_scale,
                                         int cols, int K, long lda, long sbn, long ldc, long bsA, long bsB, long bsC, int ld_scale, int scale_kind) {
  extern __shared__ __align__(16) float a_s[];
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int i = blockIdx.x, b = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const E* a = A + (size_t)b * bsA + (size_t)i * lda;
  for (int k = threadIdx.x; k < K; k += blockDim.x) a_s[k] = to_f(a[k]);
  __syncthreads();
  float s = 1.f;
  if (row_scale) {
    s = row_scale[(size_t)i * ld_scale + b];
    if (scale_kind == 2) s = 1.f / (1.f + expf(-s));
  }
  for (int j = blockIdx.z * nw + warp; j < cols; j += gridDim.z * nw) {
    const float acc = warp_dot(B + (size_t)b * bsB + (size_t)j * sbn, a_s, K, lane);
    if (lane == 0) C[(size_t)b * bsC + (size_t)i * ldc + j] = from_f<E>(acc * s);
  }
}

// gemm_batched_mma.cu
int launch_gemm_batched_mma(const bf16* A, const bf16* B, bf16* C, const float* row_scale, int rows, int cols, int K, long lda, long ldb, long ldc,
                            int batch, long bsA, long bsB, long bsC, int ld_scale, int scale_kind, cudaStream_t st);

static inline int grid_1d(long n, int block) {
  long g = (n + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

// ---- Dynamic Tanh, the norm of pre-norm blocks that computes no statistics: h = tanh(alpha * x) * w + b (alpha a scalar)
// x[t] = float(embed[ids[t]]) * scale
template <typename E>
__global__ void embed_scaled_kernel(const E* __restrict__ embed, const int* __restrict__ tok, float* __restrict__ x, int width, float scale) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x;
  const E* row = embed + (size_t)tok[t] * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) x[(size_t)t * width + i] = to_f(row[i]) * scale;
}

// x[t] += (ya[t] + yf[t]) (each optional: the sublayers of a parallel block), then h[t] = E(dyt(x[t])) and h32[t] = the same unrounded
// (few-row fp32 projections read it).  w == null: only the sum (after the last layer).
template <typename E>
__global__ void add_dyt_kernel(const E* __restrict__ ya, const float* __restrict__ yf, const float* __restrict__ alpha, const E* __restrict__ w,
                               const E* __restrict__ b, float* __restrict__ x, E* __restrict__ h, float* __restrict__ h32, long total, int width) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const float a = w ? alpha[0] : 0.f;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    float r = x[i];
    if (ya || yf) {
      const float y = (ya ? to_f(ya[i]) : 0.f) + (yf ? yf[i] : 0.f);
      r += y;
      x[i] = r;
    }
    if (w) {
      const int c = (int)(i % width);
      const float v = tanhf(a * r) * to_f(w[c]) + to_f(b[c]);
      h[i] = from_f<E>(v);
      if (h32) h32[i] = v;
    }
  }
}

// out[r] = E(dyt(x[rows[r]])): the model's last norm, only for the rows whose logits are wanted
template <typename E>
__global__ void dyt_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ alpha, const E* __restrict__ w,
                                const E* __restrict__ b, E* __restrict__ out, int width) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const float* xr = x + (size_t)rows[blockIdx.x] * width;
  const float a = alpha[0];
  for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)blockIdx.x * width + i] = from_f<E>(tanhf(a * xr[i]) * to_f(w[i]) + to_f(b[i]));
}

// out = float(in) * scale (logits of a head with an output multiplier)
template <typename A>
__global__ void scale_to_f32_kernel(const A* __restrict__ in, float* __restrict__ out, long n, float scale) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) out[i] = to_f(in[i]) * scale;
}


// ---- RMS norm in groups and "sandwich" blocks (a norm before AND after each sublayer):
//   gnorm(v, w)[i] = v[i] / sqrt(mean_{k in group(i)} v[k]^2 + eps) * w[i],  a row is `groups` equal consecutive parts.
//   x <- x + mult * gnorm((y + bias) * logistic(gate + gate_bias), w_post);   h = gnorm(x, w_next)
// One CTA per token; the row lives in shared memory as fp32, statistics and the residual sum are fp32.

// reciprocal root mean square of every group of row[0 .. width): each group is summed by `parts` warps over fixed slices and
// the slices are added in order, so the result does not depend on timing.  part_s: >= max(groups, warps) floats, inv_s: groups.
__device__ __forceinline__ void group_inv_rms(const float* row, int width, int groups, float eps, float* part_s, float* inv_s) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int gsz = width / groups, parts = nw > groups ? nw / groups : 1, items = groups * parts, slice = (gsz + parts - 1) / parts;
  __syncthreads();  // the row is complete (and nobody still reads the previous statistics)
  for (int it = warp; it < items; it += nw) {
    const int g = it / parts, pt = it % parts;
    const int lo = pt * slice, hi = min(gsz, lo + slice);
    float ss = 0.f;
    for (int i = lo + lane; i < hi; i += 32) {
      const float v = row[g * gsz + i];
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) part_s[it] = ss;
  }
  __syncthreads();
  for (int g = threadIdx.x; g < groups; g += blockDim.x) {
    float ss = 0.f;
    for (int pt = 0; pt < parts; ++pt) ss += part_s[g * parts + pt];
    inv_s[g] = 1.f / sqrtf(ss / (float)gsz + eps);
  }
  __syncthreads();
}

// eight consecutive entries at once (16-byte accesses for bf16, two for float); p must be 16-byte aligned
__device__ __forceinline__ void ld8(const bf16* p, float* o) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  o[0] = bf16_lo(v.x), o[1] = bf16_hi(v.x), o[2] = bf16_lo(v.y), o[3] = bf16_hi(v.y);
  o[4] = bf16_lo(v.z), o[5] = bf16_hi(v.z), o[6] = bf16_lo(v.w), o[7] = bf16_hi(v.w);
}
__device__ __forceinline__ void ld8(const float* p, float* o) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x, o[1] = a.y, o[2] = a.z, o[3] = a.w, o[4] = b.x, o[5] = b.y, o[6] = b.z, o[7] = b.w;
}
__device__ __forceinline__ void st8(bf16* p, const float* v) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
__device__ __forceinline__ void st8(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// logistic gate of a sublayer's result: exact in the all-fp32 build, on the fast exponential / division when activations are bf16
template <typename E>
__device__ __forceinline__ float gate_logistic(float z) {
  if constexpr (sizeof(E) == 2) return __fdividef(1.f, 1.f + __expf(-z));
  else return 1.f / (1.f + expf(-z));
}

// x[t] = gnorm(embed[ids[t]], w_embed);  h[t] = gnorm(x[t], w_next) in the element type (w_next may be null)
template <typename E>
__global__ void embed_gnorm_kernel(const E* __restrict__ embed, const int* __restrict__ tok, const E* __restrict__ w_embed, float* __restrict__ x,
                                   const E* __restrict__ w_next, E* __restrict__ h, int width, int groups, float eps) {
  extern __shared__ float gn_sm[];
  float* row = gn_sm;
  float* inv_s = row + width;
  float* part_s = inv_s + groups;
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x, gsz = width / groups;
  const E* src = embed + (size_t)tok[t] * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = to_f(src[i]);
  group_inv_rms(row, width, groups, eps, part_s, inv_s);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float r = row[i] * inv_s[i / gsz] * to_f(w_embed[i]);
    x[(size_t)t * width + i] = r;
    row[i] = r;
  }
  if (!w_next) return;
  group_inv_rms(row, width, groups, eps, part_s, inv_s);
  for (int i = threadIdx.x; i < width; i += blockDim.x) h[(size_t)t * width + i] = from_f<E>(row[i] * inv_s[i / gsz] * to_f(w_next[i]));
}

// The step between two sublayers of a sandwich block.  y [tokens, width] (E or float) is a sublayer's result, `bias` (may be null)
// its projection bias, `gate` (may be null; rows of stride gate_ld, + gate_bias) the pre-activation of its logistic gate.
template <typename E, typename Y>
__global__ void gated_gnorm_add_kernel(const Y* __restrict__ y, const E* __restrict__ bias, const E* __restrict__ gate, long gate_ld,
                                       const E* __restrict__ gate_bias, const E* __restrict__ w_post, float mult, float* __restrict__ x,
                                       const E* __restrict__ w_next, E* __restrict__ h, int width, int groups, float eps, int vec) {
  extern __shared__ float gn_sm[];
  float* row = gn_sm;
  float* inv_s = row + width;
  float* part_s = inv_s + groups;
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x, gsz = width / groups;
  if (vec) {  // width a multiple of 8 and every row 16-byte aligned: the same arithmetic on eight entries per access
    for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
      float v[8], b[8];
      ld8(y + (size_t)t * width + i, v);
      if (bias) {
        ld8(bias + i, b);
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] += b[u];
      }
      if (gate) {
        float z[8];
        ld8(gate + (size_t)t * gate_ld + i, z);
        if (gate_bias) {
          ld8(gate_bias + i, b);
#pragma unroll
          for (int u = 0; u < 8; ++u) z[u] += b[u];
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] *= gate_logistic<E>(z[u]);
      }
      st8(row + i, v);
    }
    group_inv_rms(row, width, groups, eps, part_s, inv_s);
    for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
      float xv[8], w[8], r[8];
      ld8(x + (size_t)t * width + i, xv);
      ld8(w_post + i, w);
      ld8(row + i, r);
      const float inv = inv_s[i / gsz];  // the eight entries lie in one group (gsz is a multiple of 8 on this path)
#pragma unroll
      for (int u = 0; u < 8; ++u) xv[u] += mult * (r[u] * inv * w[u]);
      st8(row + i, xv);
      st8(x + (size_t)t * width + i, xv);
    }
    if (!w_next) return;
    group_inv_rms(row, width, groups, eps, part_s, inv_s);
    for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
      float w[8], o[8], r[8];
      ld8(w_next + i, w);
      ld8(row + i, r);
      const float inv = inv_s[i / gsz];
#pragma unroll
      for (int u = 0; u < 8; ++u) o[u] = r[u] * inv * w[u];
      st8(h + (size_t)t * width + i, o);
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = to_f(y[(size_t)t * width + i]) + (bias ? to_f(bias[i]) : 0.f);
    if (gate) {
      const float z = to_f(gate[(size_t)t * gate_ld + i]) + (gate_bias ? to_f(gate_bias[i]) : 0.f);
      v *= gate_logistic<E>(z);
    }
    row[i] = v;
  }
  group_inv_rms(row, width, groups, eps, part_s, inv_s);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float r = x[(size_t)t * width + i] + mult * (row[i] * inv_s[i / gsz] * to_f(w_post[i]));
    x[(size_t)t * width + i] = r;
    row[i] = r;
  }
  if (!w_next) return;
  group_inv_rms(row, width, groups, eps, part_s, inv_s);
  for (int i = threadIdx.x; i < width; i += blockDim.x) h[(size_t)t * width + i] = from_f<E>(row[i] * inv_s[i / gsz] * to_f(w_next[i]));
}

// out[r] = gnorm(x[rows[r]], w) in the element type: the model's last norm, only for the rows whose logits are wanted
template <typename E>
__global__ void gnorm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, const E* __restrict__ w, E* __restrict__ out, int width,
                                  int groups, float eps) {
  extern __shared__ float gn_sm[];
  float* row = gn_sm;
  float* inv_s = row + width;
  float* part_s = inv_s + groups;
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const float* xr = x + (size_t)(rows ? rows[blockIdx.x] : blockIdx.x) * width;
  const int gsz = width / groups;
  for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = xr[i];
  group_inv_rms(row, width, groups, eps, part_s, inv_s);
  for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)blockIdx.x * width + i] = from_f<E>(row[i] * inv_s[i / gsz] * to_f(w[i]));
}

// ---- pre-norm blocks with plain-weight RMS norms: h = x / sqrt(mean(x^2) + eps) * w feeds a sublayer, whose result is added to x.
// A sublayer's result may be the sum of up to two branches, each optionally RMS-normed over the row with its own weight first:
//   x <- x + mult * (branch(ya, wa) + branch(yb, wb)),  branch(y, w) = w ? y / sqrt(mean(y^2) + eps) * w : y;   h = rms(x) * w_next
// One CTA per token; rows live in shared memory as fp32; sums of squares are added in a fixed order (group_inv_rms with one group).

// x[t] = embed[ids[t]] * scale;  h[t] = rms(x[t]) * w_next in the element type (and unrounded in h32 when that is not null)
template <typename E>
__global__ void embed_scaled_norm_kernel(const E* __restrict__ embed, const int* __restrict__ tok, float scale, float* __restrict__ x,
                                         const E* __restrict__ w_next, E* __restrict__ h, float* __restrict__ h32, int width, float eps) {
  extern __shared__ float gn_sm[];
  float* row = gn_sm;
  float* inv_s = row + width;
  float* part_s = inv_s + 1;
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x;
  const E* src = embed + (size_t)tok[t] * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = to_f(src[i]) * scale;
    row[i] = v;
    x[(size_t)t * width + i] = v;
  }
  if (!w_next) return;
  group_inv_rms(row, width, 1, eps, part_s, inv_s);
  const float inv = inv_s[0];
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = row[i] * inv * to_f(w_next[i]);
    h[(size_t)t * width + i] = from_f<E>(v);
    if (h32) h32[(size_t)t * width + i] = v;
  }
}

// sums of two values over the CTA, the same on every thread: lanes by shuffles, then the warps' partial sums in warp order (a fixed
// order, so a row's result does not depend on timing).  red: 64 floats of shared memory.
__device__ __forceinline__ float2 block_sum2(float a, float b, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  __syncthreads();  // the previous use of `red` has been read
  if (lane == 0) {
    red[w] = a;
    red[32 + w] = b;
  }
  __syncthreads();
  float ta = 0.f, tb = 0.f;
  for (int i = 0; i < nw; ++i) {
    ta += red[i];
    tb += red[32 + i];
  }
  return make_float2(ta, tb);
}

template <typename E, typename Y>
__global__ void branches_add_norm_kernel(const Y* __restrict__ ya, const E* __restrict__ wa, const E* __restrict__ yb, const E* __restrict__ wb, float mult,
                                         float* __restrict__ x, const E* __restrict__ w_next, E* __restrict__ h, float* __restrict__ h32, int width,
                                         float eps) {
  extern __shared__ float gn_sm[];
  float* row = gn_sm;         // branch a, then the new residual row
  float* rowb = row + width;  // branch b
  float* red = rowb + width;  // 64 floats
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x;
  const size_t at = (size_t)t * width;
  for (int i = threadIdx.x * 32; i < width; i += blockDim.x * 32) {  // what the later phases read, on its way while the sums are made
    prefetch_l2(x + at + i);
    if (wa) prefetch_l2(wa + i);
    if (wb) prefetch_l2(wb + i);
    if (w_next) prefetch_l2(w_next + i);
  }
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float a = ya ? to_f(ya[at + i]) : 0.f, b = yb ? to_f(yb[at + i]) : 0.f;
    row[i] = a;
    rowb[i] = b;
    sa = fmaf(a, a, sa);
    sb = fmaf(b, b, sb);
  }
  float inv_a = 1.f, inv_b = 1.f;
  if ((ya && wa) || (yb && wb)) {  // both branches' sums of squares in one pass
    const float2 ss = block_sum2(sa, sb, red);
    inv_a = 1.f / sqrtf(ss.x / (float)width + eps);
    inv_b = 1.f / sqrtf(ss.y / (float)width + eps);
  }
  float sr = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {  // every thread meets the entries it wrote itself
    const float a = ya ? (wa ? row[i] * inv_a * to_f(wa[i]) : row[i]) : 0.f;
    const float b = yb ? (wb ? rowb[i] * inv_b * to_f(wb[i]) : rowb[i]) : 0.f;
    const float r = x[at + i] + mult * (a + b);
    x[at + i] = r;
    row[i] = r;
    sr = fmaf(r, r, sr);
  }
  if (!w_next) return;
  const float inv = 1.f / sqrtf(block_sum2(sr, 0.f, red).x / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = row[i] * inv * to_f(w_next[i]);
    h[at + i] = from_f<E>(v);
    if (h32) h32[at + i] = v;
  }
}

// out = cap * tanh(float(in) * scale / cap)  (cap 0: float(in) * scale)
template <typename A>
__global__ void logits_scale_cap_kernel(const A* __restrict__ in, float* __restrict__ out, long n, float scale, float cap) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float z = to_f(in[i]) * scale;
    out[i] = cap > 0.f ? cap * tanhf(z / cap) : z;
  }
}

// in [T, 2F] = [gate | up]: g = min(gate, limit), u = clamp(up, -limit, limit), out = g * logistic(slope * g) * (u + 1)
template <typename E>
__global__ void act_clamped_kernel(const E* __restrict__ in, E* __restrict__ out, int F, long total, float limit, float slope) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long t = i / F, f = i % F;
    const float g = fminf(to_f(in[t * 2 * F + f]), limit), u = fminf(fmaxf(to_f(in[t * 2 * F + F + f]), -limit), limit);
    out[i] = from_f<E>(g / (1.f + expf(-slope * g)) * (u + 1.f));
  }
}

// threads per row: about two entries per thread for a few rows (every dependent round of loads costs a memory latency, and a step of
// one token is nothing but such rounds), 256 for many rows
static inline int gnorm_threads(int width, int tokens) {
  if (tokens > 64) return 256;
  const int t = (width / 2 + 31) / 32 * 32;
  return t < 128 ? 128 : t > 1024 ? 1024 : t;
}
static inline size_t gnorm_smem(int width, int groups) { return (size_t)(width + groups + std::max(groups, 32)) * sizeof(float); }
template <typename K>
static bool gnorm_fits(K kernel, size_t smem) {  // rows above 48 KB of shared memory need the opt-in limit (set once per kernel)
  if (smem <= 48 * 1024) return true;
  if (smem > 200 * 1024) return false;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess;
}

}  // namespace pk

using namespace pk;

#define PK_BY_TYPE(f32, CALL_F, CALL_B) \
  do {                                  \
    if (f32) {                          \
      CALL_F;                           \
    } else {                            \
      CALL_B;                           \
    }                                   \
  } while (0)

extern "C" int pk_res32_embed(const void* embed, const int* token_ids, float* x, void* xa, int width, int tokens, int f32, pk_stream st) {
  if (!embed || !token_ids || !x || !xa || width <= 0 || tokens <= 0) return -1;
  PK_BY_TYPE(f32, launch(embed_res32_kernel<float>, dim3(tokens), dim3(256), 0, st, true, (const float*)embed, token_ids, x, (float*)xa, width),
             launch(embed_res32_kernel<bf16>, dim3(tokens), dim3(256), 0, st, true, (const bf16*)embed, token_ids, x, (bf16*)xa, width));
  return (int)cudaGetLastError();
}

extern "C" int pk_res32_offset_norm_add(const void* y, int y_is_f32, const void* w, float* x, void* xa, int width, int tokens, float eps, int f32,
                                        pk_stream st) {
  if (!y || !w || !x || !xa || width <= 0 || tokens <= 0) return -1;
  if (f32) {
    launch(offset_norm_residual_kernel<float, float>, dim3(tokens), dim3(256), 0, st, true, (const float*)y, (const float*)w, x, (float*)xa, width, eps);
  } else if (y_is_f32) {
    launch(offset_norm_residual_kernel<bf16, float>, dim3(tokens), dim3(256), 0, st, true, (const float*)y, (const bf16*)w, x, (bf16*)xa, width, eps);
  } else {
    launch(offset_norm_residual_kernel<bf16, bf16>, dim3(tokens), dim3(256), 0, st, true, (const bf16*)y, (const bf16*)w, x, (bf16*)xa, width, eps);
  }
  return (int)cudaGetLastError();
}

extern "C" int pk_res32_offset_norm_rows(const float* x, const int* rows, const void* w, void* out, int width, int n_rows, float eps, int f32,
                                         pk_stream st) {
  if (!x || !rows || !w || !out || width <= 0 || n_rows <= 0) return -1;
  PK_BY_TYPE(f32, launch(offset_norm_rows_kernel<float>, dim3(n_rows), dim3(256), 0, st, true, x, rows, (const float*)w, (float*)out, width, eps),
             launch(offset_norm_rows_kernel<bf16>, dim3(n_rows), dim3(256), 0, st, true, x, rows, (const bf16*)w, (bf16*)out, width, eps));
  return (int)cudaGetLastError();
}

extern "C" int pk_res32_skinny_proj(const void* W, const float* x, float* out, int M, int K, int tokens, int f32, pk_stream st) {
  if (!W || !x || !out || M <= 0 || K <= 0 || tokens <= 0) return -1;
  const int threads = M >= 4 ? 128 : 32 * M;
  const dim3 grid(tokens, tokens >= 256 ? 1 : (M + 3) / 4);  // few tokens: spread the rows over CTAs
  PK_BY_TYPE(f32, launch(skinny_proj_kernel<float>, grid, dim3(threads), 0, st, true, (const float*)W, x, out, M, K),
             launch(skinny_proj_kernel<bf16>, grid, dim3(threads), 0, st, true, (const bf16*)W, x, out, M, K));
  return (int)cudaGetLastError();
}

extern "C" int pk_act(const void* in, void* out, int F, int tokens, int kind, int f32, pk_stream st) {
  if (!in || !out || F <= 0 || tokens <= 0 || kind < 0 || kind > 1) return -1;
  const long total = (long)F * tokens;
  PK_BY_TYPE(f32, launch(act_kernel<float>, dim3(grid_1d(total, 256)), dim3(256), 0, st, true, (const float*)in, (float*)out, F, total, kind),
             launch(act_kernel<bf16>, dim3(grid_1d(total, 256)), dim3(256), 0, st, true, (const bf16*)in, (bf16*)out, F, total, kind));
  return (int)cudaGetLastError();
}

extern "C" int pk_convert(const void* in, int in_f32, void* out, int out_f32, long n, pk_stream st) {
  if (!in || !out || n <= 0) return -1;
  const dim3 g(grid_1d(n, 256)), b(256);
  if (in_f32 && out_f32) launch(convert_kernel<float, float>, g, b, 0, st, true, (const float*)in, (float*)out, n);
  else if (in_f32) launch(convert_kernel<float, bf16>, g, b, 0, st, true, (const float*)in, (bf16*)out, n);
  else if (out_f32) launch(convert_kernel<bf16, float>, g, b, 0, st, true, (const bf16*)in, (float*)out, n);
  else launch(convert_kernel<bf16, bf16>, g, b, 0, st, true, (const bf16*)in, (bf16*)out, n);
  return (int)cudaGetLastError();
}

extern "C" int pk_gemm_strided(const void* A, const void* B, void* C, const float* row_scale, int rows, int cols, int K, long lda, long sbk,
                               long sbn, long ldc, int batch, long bsA, long bsB, long bsC, int ld_scale, int scale_kind, int f32, pk_stream st) {
  if (!A || !B || !C || rows <= 0 || cols <= 0 || K <= 0 || batch <= 0) return -1;
  if (rows <= 8 && sbk == 1 && K <= 8192) {
    const dim3 gr(rows, batch, (cols + 31) / 32), br(256);
    const size_t sm = (size_t)K * sizeof(float);
    PK_BY_TYPE(f32,
               launch(gemm_strided_rows_kernel<float>, gr, br, sm, st, true, (const float*)A, (const float*)B, (float*)C, row_scale, cols, K, lda, sbn,
                      ldc, bsA, bsB, bsC, ld_scale, scale_kind),
               launch(gemm_strided_rows_kernel<bf16>, gr, br, sm, st, true, (const bf16*)A, (const bf16*)B, (bf16*)C, row_scale, cols, K, lda, sbn, ldc,
                      bsA, bsB, bsC, ld_scale, scale_kind));
    return (int)cudaGetLastError();
  }
  if (!f32 && sbk == 1 && rows >= 32) {  // many rows in bf16: the tensor-core kernel when the operands are laid out for it
    const int rc = launch_gemm_batched_mma((const bf16*)A, (const bf16*)B, (bf16*)C, row_scale, rows, cols, K, lda, sbn, ldc, batch, bsA, bsB, bsC,
                                           ld_scale, scale_kind, st);
    if (rc != -2) return rc;
  }
  const dim3 g((cols + 63) / 64, (rows + 63) / 64, batch), b(256);
  PK_BY_TYPE(f32,
             launch(gemm_strided_kernel<float>, g, b, 0, st, true, (const float*)A, (const float*)B, (float*)C, row_scale, rows, cols, K, lda, sbk,
                    sbn, ldc, bsA, bsB, bsC, ld_scale, scale_kind),
             launch(gemm_strided_kernel<bf16>, g, b, 0, st, true, (const bf16*)A, (const bf16*)B, (bf16*)C, row_scale, rows, cols, K, lda, sbk, sbn,
                    ldc, bsA, bsB, bsC, ld_scale, scale_kind));
  return (int)cudaGetLastError();
}

extern "C" int pk_res32_embed_scaled(const void* embed, const int* token_ids, float* x, int width, int tokens, float scale, int f32, pk_stream st) {
  if (!embed || !token_ids || !x || width <= 0 || tokens <= 0) return -1;
  PK_BY_TYPE(f32, launch(embed_scaled_kernel<float>, dim3(tokens), dim3(256), 0, st, true, (const float*)embed, token_ids, x, width, scale),
             launch(embed_scaled_kernel<bf16>, dim3(tokens), dim3(256), 0, st, true, (const bf16*)embed, token_ids, x, width, scale));
  return (int)cudaGetLastError();
}

extern "C" int pk_res32_add_dyt(const void* ya, const float* yf, const float* alpha, const void* w, const void* b, float* x, void* h, float* h32,
                                int width, int tokens, int f32, pk_stream st) {
  if (!x || width <= 0 || tokens <= 0 || (w && (!alpha || !b || !h)) || (!w && !ya && !yf)) return -1;
  const long total = (long)width * tokens;
  PK_BY_TYPE(f32,
             launch(add_dyt_kernel<float>, dim3(grid_1d(total, 256)), dim3(256), 0, st, true, (const float*)ya, yf, alpha, (const float*)w, (const float*)b, x,
                    (float*)h, h32, total, width),
             launch(add_dyt_kernel<bf16>, dim3(grid_1d(total, 256)), dim3(256), 0, st, true, (const bf16*)ya, yf, alpha, (const bf16*)w, (const bf16*)b, x,
                    (bf16*)h, h32, total, width));
  return (int)cudaGetLastError();
}

extern "C" int pk_res32_dyt_rows(const float* x, const int* rows, const float* alpha, const void* w, const void* b, void* out, int width, int n_rows,
                                 int f32, pk_stream st) {
  if (!x || !rows || !alpha || !w || !b || !out || width <= 0 || n_rows <= 0) return -1;
  PK_BY_TYPE(f32, launch(dyt_rows_kernel<float>, dim3(n_rows), dim3(256), 0, st, true, x, rows, alpha, (const float*)w, (const float*)b, (float*)out, width),
             launch(dyt_rows_kernel<bf16>, dim3(n_rows), dim3(256), 0, st, true, x, rows, alpha, (const bf16*)w, (const bf16*)b, (bf16*)out, width));
  return (int)cudaGetLastError();
}

extern "C" int pk_scale_to_f32(const void* in, int in_f32, float* out, long n, float scale, pk_stream st) {
  if (!in || !out || n <= 0) return -1;
  const dim3 g(grid_1d(n, 256)), b(256);
  if (in_f32) launch(scale_to_f32_kernel<float>, g, b, 0, st, true, (const float*)in, out, n, scale);
  else launch(scale_to_f32_kernel<bf16>, g, b, 0, st, true, (const bf16*)in, out, n, scale);
  return (int)cudaGetLastError();
}

extern "C" int pk_res32_embed_gnorm(const void* embed, const int* token_ids, const void* w_embed, float* x, const void* w_next, void* h, int width,
                                    int groups, float eps, int tokens, int f32, pk_stream st) {
  if (!embed || !token_ids || !w_embed || !x || (w_next && !h) || width <= 0 || groups <= 0 || width % groups || tokens <= 0) return -1;
  const size_t sm = gnorm_smem(width, groups);
  if (!(f32 ? gnorm_fits(embed_gnorm_kernel<float>, sm) : gnorm_fits(embed_gnorm_kernel<bf16>, sm))) return -2;
  PK_BY_TYPE(f32,
             launch(embed_gnorm_kernel<float>, dim3(tokens), dim3(gnorm_threads(width, tokens)), sm, st, true, (const float*)embed, token_ids, (const float*)w_embed, x,
                    (const float*)w_next, (float*)h, width, groups, eps),
             launch(embed_gnorm_kernel<bf16>, dim3(tokens), dim3(gnorm_threads(width, tokens)), sm, st, true, (const bf16*)embed, token_ids, (const bf16*)w_embed, x,
                    (const bf16*)w_next, (bf16*)h, width, groups, eps));
  return (int)cudaGetLastError();
}

extern "C" int pk_res32_gated_gnorm_add(const void* y, int y_is_f32, const void* bias, const void* gate, long gate_ld, const void* gate_bias,
                                        const void* w_post, float mult, float* x, const void* w_next, void* h, int width, int groups, float eps,
                                        int tokens, int f32, pk_stream st) {
  if (!y || !w_post || !x || (w_next && !h) || width <= 0 || groups <= 0 || width % groups || tokens <= 0) return -1;
  const size_t sm = gnorm_smem(width, groups);
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const int es = f32 ? 4 : 2;
  const int vec = (width / groups) % 8 == 0 && al16(y) && al16(bias) && al16(gate) && al16(gate_bias) && al16(w_post) && al16(x) && al16(w_next) && al16(h) &&
                  (gate_ld * es) % 16 == 0;
  const int thr = vec ? std::min(gnorm_threads(width, tokens), std::max(32, (width / 8 + 31) / 32 * 32)) : gnorm_threads(width, tokens);
  const dim3 g(tokens), b(thr);
  if (f32) {
    if (!gnorm_fits(gated_gnorm_add_kernel<float, float>, sm)) return -2;
    launch(gated_gnorm_add_kernel<float, float>, g, b, sm, st, true, (const float*)y, (const float*)bias, (const float*)gate, gate_ld,
           (const float*)gate_bias, (const float*)w_post, mult, x, (const float*)w_next, (float*)h, width, groups, eps, vec);
  } else if (y_is_f32) {
    if (!gnorm_fits(gated_gnorm_add_kernel<bf16, float>, sm)) return -2;
    launch(gated_gnorm_add_kernel<bf16, float>, g, b, sm, st, true, (const float*)y, (const bf16*)bias, (const bf16*)gate, gate_ld,
           (const bf16*)gate_bias, (const bf16*)w_post, mult, x, (const bf16*)w_next, (bf16*)h, width, groups, eps, vec);
  } else {
    if (!gnorm_fits(gated_gnorm_add_kernel<bf16, bf16>, sm)) return -2;
    launch(gated_gnorm_add_kernel<bf16, bf16>, g, b, sm, st, true, (const bf16*)y, (const bf16*)bias, (const bf16*)gate, gate_ld,
           (const bf16*)gate_bias, (const bf16*)w_post, mult, x, (const bf16*)w_next, (bf16*)h, width, groups, eps, vec);
  }
  return (int)cudaGetLastError();
}

extern "C" int pk_res32_gnorm_rows(const float* x, const int* rows, const void* w, void* out, int width, int groups, float eps, int n_rows, int f32,
                                   pk_stream st) {
  if (!x || !w || !out || width <= 0 || groups <= 0 || width % groups || n_rows <= 0) return -1;
  const size_t sm = gnorm_smem(width, groups);
  if (!(f32 ? gnorm_fits(gnorm_rows_kernel<float>, sm) : gnorm_fits(gnorm_rows_kernel<bf16>, sm))) return -2;
  PK_BY_TYPE(f32, launch(gnorm_rows_kernel<float>, dim3(n_rows), dim3(gnorm_threads(width, n_rows)), sm, st, true, x, rows, (const float*)w, (float*)out, width, groups, eps),
             launch(gnorm_rows_kernel<bf16>, dim3(n_rows), dim3(gnorm_threads(width, n_rows)), sm, st, true, x, rows, (const bf16*)w, (bf16*)out, width, groups, eps));
  return (int)cudaGetLastError();
}

extern "C" int pk_res32_embed_scaled_norm(const void* embed, const int* token_ids, float scale, float* x, const void* w_next, void* h, float* h32,
                                          int width, float eps, int tokens, int f32, pk_stream st) {
  if (!embed || !token_ids || !x || (w_next && !h) || width <= 0 || tokens <= 0) return -1;
  const size_t sm = gnorm_smem(width, 1);
  if (!(f32 ? gnorm_fits(embed_scaled_norm_kernel<float>, sm) : gnorm_fits(embed_scaled_norm_kernel<bf16>, sm))) return -2;
  const dim3 g(tokens), b(gnorm_threads(width, tokens));
  PK_BY_TYPE(f32, launch(embed_scaled_norm_kernel<float>, g, b, sm, st, true, (const float*)embed, token_ids, scale, x, (const float*)w_next, (float*)h, h32, width, eps),
             launch(embed_scaled_norm_kernel<bf16>, g, b, sm, st, true, (const bf16*)embed, token_ids, scale, x, (const bf16*)w_next, (bf16*)h, h32, width, eps));
  return (int)cudaGetLastError();
}

extern "C" int pk_res32_branches_add_norm(const void* ya, int ya_is_f32, const void* wa, const void* yb, const void* wb, float mult, float* x,
                                          const void* w_next, void* h, float* h32, int width, float eps, int tokens, int f32, pk_stream st) {
  if (!x || (w_next && !h) || width <= 0 || tokens <= 0) return -1;
  const size_t sm = (size_t)(2 * width + 64) * sizeof(float);
  const dim3 g(tokens), b(gnorm_threads(width, tokens));
  if (f32) {
    if (!gnorm_fits(branches_add_norm_kernel<float, float>, sm)) return -2;
    launch(branches_add_norm_kernel<float, float>, g, b, sm, st, true, (const float*)ya, (const float*)wa, (const float*)yb, (const float*)wb, mult, x,
           (const float*)w_next, (float*)h, h32, width, eps);
  } else if (ya_is_f32) {
    if (!gnorm_fits(branches_add_norm_kernel<bf16, float>, sm)) return -2;
    launch(branches_add_norm_kernel<bf16, float>, g, b, sm, st, true, (const float*)ya, (const bf16*)wa, (const bf16*)yb, (const bf16*)wb, mult, x,
           (const bf16*)w_next, (bf16*)h, h32, width, eps);
  } else {
    if (!gnorm_fits(branches_add_norm_kernel<bf16, bf16>, sm)) return -2;
    launch(branches_add_norm_kernel<bf16, bf16>, g, b, sm, st, true, (const bf16*)ya, (const bf16*)wa, (const bf16*)yb, (const bf16*)wb, mult, x,
           (const bf16*)w_next, (bf16*)h, h32, width, eps);
  }
  return (int)cudaGetLastError();
}

extern "C" int pk_logits_scale_cap(const void* in, int in_f32, float* out, long n, float scale, float cap, pk_stream st) {
  if (!in || !out || n <= 0 || cap < 0.f) return -1;
  const dim3 g(grid_1d(n, 256)), b(256);
  if (in_f32) launch(logits_scale_cap_kernel<float>, g, b, 0, st, true, (const float*)in, out, n, scale, cap);
  else launch(logits_scale_cap_kernel<bf16>, g, b, 0, st, true, (const bf16*)in, out, n, scale, cap);
  return (int)cudaGetLastError();
}

extern "C" int pk_act_clamped(const void* in, void* out, int F, int tokens, float limit, float slope, int f32, pk_stream st) {
  if (!in || !out || F <= 0 || tokens <= 0 || !(limit > 0.f)) return -1;
  const long total = (long)F * tokens;
  PK_BY_TYPE(f32, launch(act_clamped_kernel<float>, dim3(grid_1d(total, 256)), dim3(256), 0, st, true, (const float*)in, (float*)out, F, total, limit, slope),
             launch(act_clamped_kernel<bf16>, dim3(grid_1d(total, 256)), dim3(256), 0, st, true, (const bf16*)in, (bf16*)out, F, total, limit, slope));
  return (int)cudaGetLastError();
}
