// Mixture-of-experts feed-forward for many tokens at once (prompt portions): the (token, choice) pairs are bucketed by
// expert, and each expert's rows run as one tensor-core GEMM over that expert's weights, so a weight tile is read once
// per 64 rows instead of once per token (moe.cu is the per-token form for a few tokens).
//   1. moe_bucket_kernel     one CTA: histogram of the routed ids, offsets per expert, a slot for every pair, and the list
//                            of 64-row tiles (expert, first slot).  Which slot a pair gets inside its expert's run may
//                            vary from run to run; every row's result is independent of its slot, so outputs do not.
//   2. moe_grouped_gemm<0>   hid[slot] = relu(W_up[e] x[token(slot)])^2          (rows gathered through the slot list)
//      moe_grouped_gemm<2>   hid[slot] = silu(W_gate[e] x) * (W_up[e] x)            (gated experts, gate / up rows interleaved)
//      moe_grouped_gemm<3>   hid[slot] = g logistic(p1 g) (u + 1), g = min(W_gate[e] x, p0), u = clamp(W_up[e] x, -p0, p0)
//   3. moe_grouped_gemm<1>   part[slot] = weight(pair) * W_down[e] hid[slot]     (fp32)
//   4. moe_combine_kernel    y[t] = sum_k part[slot(t, k)] (+ logistic(g_t) * shared[t]), summed in the order of k
// GEMM tiles: 64 rows x 64 outputs x 64 deep, 4 warps of 32 x 32, mma.sync m16n8k16 bf16 with fp32 accumulation, operands
// through a two-stage cp.async ring.  Tensor-bound: 4 * pairs * ff * width flop per layer.
#include "common.cuh"
#include "mma.cuh"

namespace pk {

constexpr int kGT = 64, kGK = 64, kGLd = kGK + 8, kGPieces = kGT * kGK / 8 / 128;  // 16-byte pieces per thread, operand and k tile

// meta layout (ints): [0] number of row tiles, [1 .. E+1] offsets (exclusive scan, E + 1 entries), then tile_expert[max_tiles],
// tile_row0[max_tiles]; slot_pair[pairs] and pair_slot[pairs] are separate arrays.
__global__ void moe_bucket_kernel(const int* __restrict__ ids, int pairs, int experts, int max_tiles, int* __restrict__ meta,
                                  int* __restrict__ slot_pair, int* __restrict__ pair_slot) {
  extern __shared__ int sh[];  // [experts] counts, then [experts] cursors
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  int* cnt = sh;
  int* cur = sh + experts;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&cnt[ids[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int* off = meta + 1;
    int* te = meta + 2 + experts;
    int* tr = te + max_tiles;
    int run = 0, nt = 0;
    for (int e = 0; e < experts; ++e) {
      off[e] = run;
      cur[e] = run;
      for (int r = 0; r < cnt[e]; r += kGT) {
        te[nt] = e;
        tr[nt] = run + r;
        ++nt;
      }
      run += cnt[e];
    }
    off[experts] = run;
    meta[0] = nt;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int s = atomicAdd(&cur[ids[p]], 1);
    slot_pair[s] = p;
    pair_slot[p] = s;
  }
}

// EPI 0: out bf16 [slots][N] = relu(acc)^2.   EPI 1: out fp32 [slots][N] = acc * weights[pair of the slot].
// EPI 2: W rows interleaved (2f = gate f, 2f + 1 = up f): out bf16 [slots][N / 2] = silu(acc[2f]) * acc[2f + 1].
// EPI 3: the same rows with clamped pre-activations: g = min(acc[2f], p0), u = clamp(acc[2f + 1], -p0, p0), out = g logistic(p1 g) (u + 1).
// A row of slot s: A + (gather_div ? slot_pair[s] / gather_div : s) * K.
template <int EPI>
__global__ void __launch_bounds__(128) moe_grouped_gemm_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, void* __restrict__ out,
                                                              const int* __restrict__ meta, const int* __restrict__ slot_pair,
                                                              const float* __restrict__ weights, int experts, int max_tiles, int N, int K,
                                                              int gather_div, float p0, float p1) {
  __shared__ __align__(16) bf16 As[2][kGT * kGLd];
  __shared__ __align__(16) bf16 Bs[2][kGT * kGLd];
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  if ((int)blockIdx.y >= meta[0]) return;
  const int* off = meta + 1;
  const int e = meta[2 + experts + blockIdx.y], m0 = meta[2 + experts + max_tiles + blockIdx.y];
  const int m_end = off[e + 1], n0 = blockIdx.x * kGT;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tq = lane & 3, wm = warp >> 1, wn = warp & 1;
  const bf16* We = W + (size_t)e * N * K;
  // each thread copies kGPieces 16-byte pieces of A and of B per k tile
  const bf16* a_src[kGPieces];
  const bf16* b_src[kGPieces];
  int kc[kGPieces], sm_off[kGPieces];
#pragma unroll
  for (int i = 0; i < kGPieces; ++i) {
    const int c = tid + i * 128, r = c / (kGK / 8);
    kc[i] = (c % (kGK / 8)) * 8;
    sm_off[i] = r * kGLd + kc[i];
    const int s = m0 + r;
    a_src[i] = s < m_end ? A + (size_t)(gather_div ? slot_pair[s] / gather_div : s) * K : nullptr;
    b_src[i] = n0 + r < N ? We + (size_t)(n0 + r) * K : nullptr;
  }
  auto load = [&](int kt, int buf) {
#pragma unroll
    for (int i = 0; i < kGPieces; ++i) {
      const int k = kt * kGK + kc[i];
      if (a_src[i] && k < K) cp_async16(&As[buf][sm_off[i]], a_src[i] + k);
      else *reinterpret_cast<uint4*>(&As[buf][sm_off[i]]) = make_uint4(0, 0, 0, 0);
      if (b_src[i] && k < K) cp_async16(&Bs[buf][sm_off[i]], b_src[i] + k);
      else *reinterpret_cast<uint4*>(&Bs[buf][sm_off[i]]) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
  };
  float acc[2][4][4] = {};
  const int nk = (K + kGK - 1) / kGK;
  load(0, 0);
  for (int kt = 0; kt < nk; ++kt) {
    const int buf = kt & 1;
    cp_async_wait_all();
    __syncthreads();
    if (kt + 1 < nk) load(kt + 1, buf ^ 1);
#pragma unroll
    for (int kk = 0; kk < kGK; kk += 16) {
      uint32_t a[2][4], b[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
        ldsm_x4(a[mi], &As[buf][(wm * 32 + mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kGLd + kk + ((lane >> 4) & 1) * 8]);
#pragma unroll
      for (int np = 0; np < 2; ++np)
        ldsm_x4(b[np], &Bs[buf][(wn * 32 + np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * kGLd + kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) mma_bf16_16816(acc[mi][ni], a[mi], b[ni >> 1][(ni & 1) * 2], b[ni >> 1][(ni & 1) * 2 + 1]);
    }
  }
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int s = m0 + wm * 32 + mi * 16 + g + hf * 8;
      if (s >= m_end) continue;
      const float wgt = EPI == 1 ? weights[slot_pair[s]] : 1.f;
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) {
        const int n = n0 + wn * 32 + ni * 8 + 2 * tq;
        float v0 = acc[mi][ni][hf * 2], v1 = acc[mi][ni][hf * 2 + 1];
        if (EPI == 0) {
          v0 = fmaxf(v0, 0.f);
          v1 = fmaxf(v1, 0.f);
          bf16* o = static_cast<bf16*>(out) + (size_t)s * N + n;
          if (n + 1 < N) *reinterpret_cast<uint32_t*>(o) = pack_bf16(v0 * v0, v1 * v1);
          else if (n < N) o[0] = f2bf(v0 * v0);
        } else if (EPI == 2) {
          if (n + 1 < N) static_cast<bf16*>(out)[(size_t)s * (N / 2) + n / 2] = f2bf(v0 / (1.f + expf(-v0)) * v1);
        } else if (EPI == 3) {
          v0 = fminf(v0, p0);
          v1 = fminf(fmaxf(v1, -p0), p0);
          if (n + 1 < N) static_cast<bf16*>(out)[(size_t)s * (N / 2) + n / 2] = f2bf(v0 / (1.f + expf(-p1 * v0)) * (v1 + 1.f));
        } else {
          float* o = static_cast<float*>(out) + (size_t)s * N + n;
          if (n + 1 < N) *reinterpret_cast<float2*>(o) = make_float2(v0 * wgt, v1 * wgt);
          else if (n < N) o[0] = v0 * wgt;
        }
      }
    }
}

__global__ void moe_combine_kernel(const float* __restrict__ part, const int* __restrict__ pair_slot, const bf16* __restrict__ shared,
                                   const float* __restrict__ sg, float* __restrict__ y, int width, int top) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int t = blockIdx.x;
  const float g = shared ? (sg ? 1.f / (1.f + expf(-sg[t])) : 1.f) : 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) acc += part[(size_t)pair_slot[(size_t)t * top + k] * width + i];
    y[(size_t)t * width + i] = acc + (shared ? g * bf2f(shared[(size_t)t * width + i]) : 0.f);
  }
}

}  // namespace pk

using namespace pk;

extern "C" long pk_moe_grouped_workspace_bytes(int tokens, int top, int experts, int width, int ff) {
  const long pairs = (long)tokens * top, max_tiles = pairs / kGT + experts + 1;
  long b = (2 + experts + 2 * max_tiles + 2 * pairs) * 4;  // meta, slot_pair, pair_slot
  b = (b + 255) / 256 * 256;
  b += (pairs * ff * 2 + 255) / 256 * 256;  // hid
  b += pairs * width * 4;                   // part
  return b + 256;
}

// y [tokens, width] fp32 = routed experts (+ gated shared expert); bf16 operands; width % 8 == 0 and ff % 8 == 0.
extern "C" int pk_moe_grouped_act(const void* xa, const void* w_up, const void* w_down, const int* ids, const float* weights, const void* shared,
                                  const float* shared_gate, float* y, void* workspace, int tokens, int top, int experts, int width, int ff, int act,
                                  pk_stream st) {
  if (act < 0 || act > 1) return -1;
  return pk_moe_grouped_act_p(xa, w_up, w_down, ids, weights, shared, shared_gate, y, workspace, tokens, top, experts, width, ff, act, 0.f, 0.f, st);
}

// act 2: clamped gated experts (limit p0, slope p1); shared_gate may be NULL with a shared expert (added without a gate)
extern "C" int pk_moe_grouped_act_p(const void* xa, const void* w_up, const void* w_down, const int* ids, const float* weights, const void* shared,
                                    const float* shared_gate, float* y, void* workspace, int tokens, int top, int experts, int width, int ff, int act,
                                    float p0, float p1, pk_stream st) {
  if (!xa || !w_up || !w_down || !ids || !weights || !y || !workspace || tokens <= 0 || top <= 0 || experts <= 0 || experts > 4096 || act < 0 || act > 2 ||
      (act == 2 && !(p0 > 0.f)))
    return -1;
  if (width % 8 || ff % 8 || (reinterpret_cast<uintptr_t>(xa) & 15) || (reinterpret_cast<uintptr_t>(w_up) & 15) ||
      (reinterpret_cast<uintptr_t>(w_down) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return -2;
  const long pairs = (long)tokens * top;
  const int max_tiles = (int)(pairs / kGT) + experts + 1;
  char* ws = static_cast<char*>(workspace);
  int* meta = reinterpret_cast<int*>(ws);
  int* slot_pair = meta + 2 + experts + 2 * max_tiles;
  int* pair_slot = slot_pair + pairs;
  long o = ((2 + experts + 2 * (long)max_tiles + 2 * pairs) * 4 + 255) / 256 * 256;
  bf16* hid = reinterpret_cast<bf16*>(ws + o);
  o += (pairs * ff * 2 + 255) / 256 * 256;
  float* part = reinterpret_cast<float*>(ws + o);
  launch(moe_bucket_kernel, dim3(1), dim3(1024), (size_t)2 * experts * sizeof(int), st, true, ids, (int)pairs, experts, max_tiles, meta, slot_pair,
         pair_slot);
  if (act == 2)
    launch(moe_grouped_gemm_kernel<3>, dim3((2 * ff + kGT - 1) / kGT, max_tiles), dim3(128), 0, st, true, (const bf16*)xa, (const bf16*)w_up, (void*)hid,
           (const int*)meta, (const int*)slot_pair, weights, experts, max_tiles, 2 * ff, width, top, p0, p1);
  else if (act == 1)
    launch(moe_grouped_gemm_kernel<2>, dim3((2 * ff + kGT - 1) / kGT, max_tiles), dim3(128), 0, st, true, (const bf16*)xa, (const bf16*)w_up, (void*)hid,
           (const int*)meta, (const int*)slot_pair, weights, experts, max_tiles, 2 * ff, width, top, 0.f, 0.f);
  else
    launch(moe_grouped_gemm_kernel<0>, dim3((ff + kGT - 1) / kGT, max_tiles), dim3(128), 0, st, true, (const bf16*)xa, (const bf16*)w_up, (void*)hid,
           (const int*)meta, (const int*)slot_pair, weights, experts, max_tiles, ff, width, top, 0.f, 0.f);
  launch(moe_grouped_gemm_kernel<1>, dim3((width + kGT - 1) / kGT, max_tiles), dim3(128), 0, st, true, (const bf16*)hid, (const bf16*)w_down,
         (void*)part, (const int*)meta, (const int*)slot_pair, weights, experts, max_tiles, width, ff, 0, 0.f, 0.f);
  launch(moe_combine_kernel, dim3(tokens), dim3(256), 0, st, true, (const float*)part, (const int*)pair_slot, (const bf16*)shared, shared_gate, y, width,
         top);
  return (int)cudaGetLastError();
}

extern "C" int pk_moe_grouped_relu2(const void* xa, const void* w_up, const void* w_down, const int* ids, const float* weights, const void* shared,
                                    const float* shared_gate, float* y, void* workspace, int tokens, int top, int experts, int width, int ff,
                                    pk_stream st) {
  return pk_moe_grouped_act(xa, w_up, w_down, ids, weights, shared, shared_gate, y, workspace, tokens, top, experts, width, ff, 0, st);
}
