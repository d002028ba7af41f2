// Latent attention over a paged cache of compressed keys/values (one latent vector c [rank] and one rotated key part
// kr [rot] per token, shared by all heads), in the "absorbed" form:
//     score(t, h, j) = (qa[t,h,:rank] . c_j + qa[t,h,rank:] . kr_j) * scale,     qa[t,h,:rank] = W_uk[h]^T q_unrotated[t,h]
//     o_lat[t,h]     = sum_j p(t,h,j) c_j,                                       head output = W_uv[h] o_lat[t,h]
// so neither keys nor values are ever expanded per head: every head reads the same [rank + rot] cache line (the KV
// traffic of multi-query attention).  The softmax denominator carries one extra term exp(sink_h) (a learned logit with
// no key and no value; sink == NULL leaves it out); the mask is causal by position, optionally limited to a sliding
// window (keys p - window + 1 .. p).  A ragged batch (portions of prompts beside single decoded
// tokens) is one launch: every query row carries its request and position.
//
// Kernels here: rotate-half rotary embedding of a slice of each head from a frequency table (any frequency schedule:
// the host builds the table, e.g. YaRN-blended), append of (normed latent, rotated key part) into the paged cache, and
// the attention itself (generic widths, fp32 arithmetic; element type bf16 or float).
// Cache layout: page p of owner layer l at base + p * page_stride + layer_off(l); inside, slot s at s * (rank + rot).
#include <cstring>

#include "common.cuh"
#include "typed.cuh"

namespace pk {

// out[t, h, out_off + i] = rotated in[t, h, in_off + i] for i < width: the first `dims` entries rotate in pairs
// (i, i + dims/2) -- or (2i, 2i + 1) when `interleaved` -- by angle pos[t] * freq[i], cos and sin times `mag`; entries
// dims..width-1 pass unchanged.

// entry i (< dims) of a rotated vector read through `at(k)`; k0 = index of the pair's frequency
template <typename F>
__device__ __forceinline__ float rotate_entry(F at, int i, int dims, int interleaved, float p, const float* __restrict__ freq, float mag) {
  const int half = dims >> 1;
  int k, first_i, second_i;
  bool first;
  if (interleaved) {
    k = i >> 1;
    first = (i & 1) == 0;
    first_i = 2 * k;
    second_i = 2 * k + 1;
  } else {
    first = i < half;
    k = first ? i : i - half;
    first_i = k;
    second_i = k + half;
  }
  const float a = p * freq[k];
  const float c = cosf(a) * mag, s = sinf(a) * mag;
  const float u = at(first_i), v = at(second_i);
  return first ? u * c - v * s : v * c + u * s;
}

template <typename E>
__global__ void rope_slice_kernel(const E* __restrict__ in, E* __restrict__ out, const int* __restrict__ pos, const float* __restrict__ freq,
                                  float mag, int heads, int in_stride, int in_off, int out_stride, int out_off, int width, int dims, int interleaved) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x;
  const float p = (float)pos[t];
  for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < heads * width; e += gridDim.y * blockDim.x) {
    const int h = e / width, i = e % width;
    const E* src = in + ((size_t)t * heads + h) * in_stride + in_off;
    const float r = i < dims ? rotate_entry([&](int k) { return to_f(src[k]); }, i, dims, interleaved, p, freq, mag) : to_f(src[i]);
    out[((size_t)t * heads + h) * out_stride + out_off + i] = from_f<E>(r);
  }
}

// One token per block: d = dkv[t] (rank + rot values).  c = d[:rank] / rms * norm_w -> cache; kr = rotate(d[rank:]) -> cache.
template <typename E>
__global__ void latent_kv_append_kernel(const E* __restrict__ dkv, const E* __restrict__ norm_w, const int* __restrict__ pos,
                                        const int* __restrict__ req, const int* __restrict__ page_off, const int* __restrict__ pages,
                                        E* __restrict__ cache, long page_stride, int page_size, int rank, int rot, int dims,
                                        const float* __restrict__ freq, float mag, float eps, int interleaved) {
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x, p = pos[t];
  const E* d = dkv + (size_t)t * (rank + rot);
  E* dst = cache + (size_t)pages[page_off[req[t]] + p / page_size] * page_stride + (size_t)(p % page_size) * (rank + rot);
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_f(d[i]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)rank + eps);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f<E>(to_f(d[i]) * inv * to_f(norm_w[i]));
  const float pf = (float)p;
  for (int i = threadIdx.x; i < rot; i += blockDim.x) {
    const float r = i < dims ? rotate_entry([&](int k) { return to_f(d[rank + k]); }, i, dims, interleaved, pf, freq, mag) : to_f(d[rank + i]);
    dst[rank + i] = from_f<E>(r);
  }
}

constexpr int kLatentMaxPerLane = 32;  // rank <= 1024

// Generic-width kernel: one block per (query row, head); warps stride over the visible keys with an online softmax each,
// lanes split the feature axis; the per-warp states and the sink are merged at the end.
template <typename E>
__global__ void latent_attention_kernel(const E* __restrict__ qa, const E* __restrict__ cache, const E* __restrict__ sink,
                                        const int* __restrict__ pos, const int* __restrict__ req, const int* __restrict__ page_off,
                                        const int* __restrict__ pages, E* __restrict__ out, long page_stride, int page_size, int heads,
                                        int rank, int rot, float scale, int window) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x, h = blockIdx.y, D = rank + rot;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float* q_s = sm;                 // [D]
  float* m_s = q_s + D;            // [nw]
  float* l_s = m_s + nw;           // [nw]
  float* acc_s = l_s + nw;         // [nw][rank]
  const E* q = qa + ((size_t)t * heads + h) * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) q_s[i] = to_f(q[i]) * scale;
  __syncthreads();
  const int p = pos[t];
  const int* pg = pages + page_off[req[t]];
  float m = -INFINITY, l = 0.f, acc[kLatentMaxPerLane];
#pragma unroll
  for (int u = 0; u < kLatentMaxPerLane; ++u) acc[u] = 0.f;
  for (int j = (window > 0 ? max(p - window + 1, 0) : 0) + warp; j <= p; j += nw) {
    const E* kv = cache + (size_t)pg[j / page_size] * page_stride + (size_t)(j % page_size) * D;
    float cv[kLatentMaxPerLane];
    float s = 0.f;
#pragma unroll
    for (int u = 0; u < kLatentMaxPerLane; ++u) {
      const int d = u * 32 + lane;
      cv[u] = d < rank ? to_f(kv[d]) : 0.f;
      if (d < rank) s = fmaf(q_s[d], cv[u], s);
    }
    for (int d = rank + lane; d < D; d += 32) s = fmaf(q_s[d], to_f(kv[d]), s);
    s = warp_sum(s);
    const float mn = fmaxf(m, s);
    const float corr = expf(m - mn), pj = expf(s - mn);
    l = l * corr + pj;
#pragma unroll
    for (int u = 0; u < kLatentMaxPerLane; ++u) acc[u] = acc[u] * corr + pj * cv[u];
    m = mn;
  }
  if (lane == 0) {
    m_s[warp] = m;
    l_s[warp] = l;
  }
#pragma unroll
  for (int u = 0; u < kLatentMaxPerLane; ++u) {
    const int d = u * 32 + lane;
    if (d < rank) acc_s[(size_t)warp * rank + d] = acc[u];
  }
  __syncthreads();
  const float sk = sink ? to_f(sink[h]) : -INFINITY;
  float M = sk;
  for (int w = 0; w < nw; ++w) M = fmaxf(M, m_s[w]);
  float den = sink ? expf(sk - M) : 0.f;
  for (int w = 0; w < nw; ++w) den += m_s[w] == -INFINITY ? 0.f : l_s[w] * expf(m_s[w] - M);
  const float inv = 1.f / den;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float o = 0.f;
    for (int w = 0; w < nw; ++w) o += m_s[w] == -INFINITY ? 0.f : acc_s[(size_t)w * rank + d] * expf(m_s[w] - M);
    out[((size_t)t * heads + h) * rank + d] = from_f<E>(o * inv);
  }
}

// latent_attention_mma.cu: tensor-core kernel for bf16 with rank % 64 == 0 and rot % 16 == 0; -2 = not for this shape
int launch_latent_attention_mma(const bf16* qa, const bf16* cache, const bf16* sink, const int* pos, const int* req, const int* page_off,
                                const int* pages, bf16* out, long page_stride, int page_size, int tokens, int heads, int rank, int rot, float scale,
                                int window, int max_kv_len, cudaStream_t st);
static bool latent_mma_enabled() {  // PK_LATENT_ATTN=generic keeps the generic kernel for A/B runs
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("PK_LATENT_ATTN");
    v = (e && strcmp(e, "generic") == 0) ? 0 : 1;
  }
  return v == 1;
}

}  // namespace pk

using namespace pk;

extern "C" int pk_rope_slice(const void* in, void* out, const int* positions, const float* freq, float mag, int tokens, int heads, int in_stride,
                             int in_off, int out_stride, int out_off, int width, int dims, int f32, pk_stream st) {
  return pk_rope_slice_ex(in, out, positions, freq, mag, tokens, heads, in_stride, in_off, out_stride, out_off, width, dims, 0, f32, st);
}

extern "C" int pk_rope_slice_ex(const void* in, void* out, const int* positions, const float* freq, float mag, int tokens, int heads, int in_stride,
                                int in_off, int out_stride, int out_off, int width, int dims, int interleaved, int f32, pk_stream st) {
  if (!in || !out || !positions || (dims > 0 && !freq) || tokens <= 0 || heads <= 0 || width <= 0 || dims < 0 || dims > width || (dims & 1)) return -1;
  const dim3 rope_grid(tokens, tokens >= 64 ? 1 : (heads * width + 127) / 128);  // few tokens: spread one token over CTAs
  if (f32)
    launch(rope_slice_kernel<float>, rope_grid, dim3(128), 0, st, true, (const float*)in, (float*)out, positions, freq, mag, heads, in_stride,
           in_off, out_stride, out_off, width, dims, interleaved);
  else
    launch(rope_slice_kernel<bf16>, rope_grid, dim3(128), 0, st, true, (const bf16*)in, (bf16*)out, positions, freq, mag, heads, in_stride, in_off,
           out_stride, out_off, width, dims, interleaved);
  return (int)cudaGetLastError();
}

extern "C" int pk_latent_kv_append(const void* dkv, const void* norm_w, const int* positions, const int* req, const int* page_off, const int* pages,
                                   void* cache, long page_stride, int page_size, int rank, int rot, int dims, const float* freq, float mag,
                                   float eps, int tokens, int f32, pk_stream st) {
  return pk_latent_kv_append_ex(dkv, norm_w, positions, req, page_off, pages, cache, page_stride, page_size, rank, rot, dims, 0, freq, mag, eps, tokens,
                                f32, st);
}

extern "C" int pk_latent_kv_append_ex(const void* dkv, const void* norm_w, const int* positions, const int* req, const int* page_off, const int* pages,
                                      void* cache, long page_stride, int page_size, int rank, int rot, int dims, int interleaved, const float* freq,
                                      float mag, float eps, int tokens, int f32, pk_stream st) {
  if (!dkv || !norm_w || !positions || !req || !page_off || !pages || !cache || (dims > 0 && !freq) || tokens <= 0 || rank <= 0 || rot < 0 || dims < 0 ||
      dims > rot || (dims & 1) || page_size <= 0)
    return -1;
  if (f32)
    launch(latent_kv_append_kernel<float>, dim3(tokens), dim3(128), 0, st, true, (const float*)dkv, (const float*)norm_w, positions, req, page_off,
           pages, (float*)cache, page_stride, page_size, rank, rot, dims, freq, mag, eps, interleaved);
  else
    launch(latent_kv_append_kernel<bf16>, dim3(tokens), dim3(128), 0, st, true, (const bf16*)dkv, (const bf16*)norm_w, positions, req, page_off,
           pages, (bf16*)cache, page_stride, page_size, rank, rot, dims, freq, mag, eps, interleaved);
  return (int)cudaGetLastError();
}

extern "C" int pk_latent_attention(const void* qa, const void* cache, const void* sink, const int* positions, const int* req, const int* page_off,
                                   const int* pages, void* out, long page_stride, int page_size, int tokens, int heads, int rank, int rot,
                                   float scale, int max_kv_len, int f32, pk_stream st) {
  if (!sink) return -1;
  return pk_latent_attention_ex(qa, cache, sink, positions, req, page_off, pages, out, page_stride, page_size, tokens, heads, rank, rot, scale, 0,
                                max_kv_len, f32, st);
}

extern "C" int pk_latent_attention_ex(const void* qa, const void* cache, const void* sink, const int* positions, const int* req, const int* page_off,
                                      const int* pages, void* out, long page_stride, int page_size, int tokens, int heads, int rank, int rot,
                                      float scale, int window, int max_kv_len, int f32, pk_stream st) {
  if (!qa || !cache || !positions || !req || !page_off || !pages || !out || tokens <= 0 || heads <= 0 || rank <= 0 || rot < 0 || window < 0) return -1;
  if (!f32 && latent_mma_enabled()) {
    const int rc = launch_latent_attention_mma((const bf16*)qa, (const bf16*)cache, (const bf16*)sink, positions, req, page_off, pages, (bf16*)out,
                                               page_stride, page_size, tokens, heads, rank, rot, scale, window, max_kv_len, st);
    if (rc != -2) return rc;
  }
  if (rank > 32 * kLatentMaxPerLane) return -2;
  const int threads = 128, nw = threads / 32;
  const size_t smem = (size_t)(rank + rot + 2 * nw + nw * rank) * sizeof(float);
  if (f32)
    launch(latent_attention_kernel<float>, dim3(tokens, heads), dim3(threads), smem, st, true, (const float*)qa, (const float*)cache,
           (const float*)sink, positions, req, page_off, pages, (float*)out, page_stride, page_size, heads, rank, rot, scale, window);
  else
    launch(latent_attention_kernel<bf16>, dim3(tokens, heads), dim3(threads), smem, st, true, (const bf16*)qa, (const bf16*)cache, (const bf16*)sink,
           positions, req, page_off, pages, (bf16*)out, page_stride, page_size, heads, rank, rot, scale, window);
  return (int)cudaGetLastError();
}
