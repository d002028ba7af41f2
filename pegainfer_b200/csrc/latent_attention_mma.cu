// Tensor-core kernel for the absorbed latent attention (see latent_attention.cu for the math and the cache layout), bf16.
// All heads read the same cache line [c_j | kr_j], so the query rows of a tile are 16 consecutive (token, head) pairs of
// the flattened [tokens * heads] axis: a prompt portion fills tiles with many tokens' heads, a decoded token's heads are
// one tile -- the same kernel serves both, and long contexts of few rows are split over the key axis (grid.y) and merged.
//
// CTA = 4 warps, 16 query rows, key tiles of 64 fetched with cp.async into a two-stage ring:
//   S   = Q K^T   warp w owns keys [16w, 16w+16) of the tile over the whole feature axis (mma.sync m16n8k16, fp32 acc)
//   row maxima / sums are exchanged through shared memory, P (bf16) goes to shared memory
//   O  += P V     V = the first `rank` columns of the same key tile; warp w owns output columns [w*rank/4, (w+1)*rank/4)
// A tile whose rows belong to several requests walks each request's keys in turn with the other rows masked (their
// accumulators see p = 0 and a correction of 1).  The sink enters once, at the end (or in the merge of the splits).
// Tensor-bound for prompt portions (2 * rows * keys * (2 rank + rot) flop), HBM/L2-bound for decode (keys * (rank + rot) * 2 B).
#include "common.cuh"
#include "mma.cuh"

namespace pk {

constexpr int kMmaKeys = 64;
constexpr float kNegBig = -1e30f;

// NV = 8-column output tiles per warp (rank = 32 * nv with nv <= NV, nv even); MT = 16-row query tiles per warp group;
// WG = groups of 4 warps, each with its own MT tiles, sharing the fetched key tiles (2 for prompt portions: twice the rows per
// key fetch and two warps per scheduler to hide each other's latencies; 1 for the few rows of a decode step)
template <int NV, int MT, int WG>
__global__ void __launch_bounds__(128 * WG)
latent_attention_mma_kernel(const bf16* __restrict__ qa, const bf16* __restrict__ cache, const bf16* __restrict__ sink, const int* __restrict__ pos,
                            const int* __restrict__ req, const int* __restrict__ page_off, const int* __restrict__ pages, bf16* __restrict__ out,
                            float* __restrict__ part_o, float* __restrict__ part_ml, long page_stride, int page_size, int tokens, int heads, int rank,
                            int rot, float scale, int window) {
  constexpr int ROWS_G = 16 * MT, ROWS = ROWS_G * WG, NR = 2 * MT;  // NR = rows per thread: rb + g + 8 * i, i < NR
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = rank + rot, ldk = D + 8, nv = rank / 32;
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);   // [ROWS][ldk]
  bf16* Ks = Qs + ROWS * ldk;                     // [2][64][ldk]
  bf16* Ps = Ks + 2 * kMmaKeys * ldk;             // [ROWS][72]
  float* wmax = reinterpret_cast<float*>(Ps + ROWS * 72);  // [4][ROWS]
  float* wsum = wmax + 4 * ROWS;                           // [4][ROWS]
  const int tid = threadIdx.x, lane = tid & 31, warp = (tid >> 5) & 3, rb = (tid >> 7) * ROWS_G, g = lane >> 2, tq = lane & 3;
  const int nthreads = 128 * WG;
  const int total_rows = tokens * heads, R0 = blockIdx.x * ROWS;
  const int split = blockIdx.y, nsplit = gridDim.y;
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads

  // ---- Q tile (rows past the end are zero)
  const int chunks = D / 8;  // 16-byte pieces per row
  for (int e = tid; e < ROWS * chunks; e += nthreads) {
    const int r = e / chunks, c = e % chunks;
    bf16* dst = Qs + r * ldk + c * 8;
    if (R0 + r < total_rows) cp_async16(dst, qa + (size_t)(R0 + r) * D + c * 8);
    else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
  }
  cp_async_commit();

  const int ld_r0 = tid / chunks, ld_c0 = tid % chunks, ld_dr = nthreads / chunks, ld_dc = nthreads % chunks;
  const int ps_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
  int row_tok[NR], row_pos[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int R = R0 + rb + g + 8 * i;
    row_tok[i] = R < total_rows ? R / heads : -1;
    row_pos[i] = row_tok[i] >= 0 ? pos[row_tok[i]] : -1;
  }
  float m_run[NR], l_run[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    m_run[i] = kNegBig;
    l_run[i] = 0.f;
  }
  float o[MT][NV][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < NV; ++i) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f;

  const int t_first = R0 / heads, t_last = (min(total_rows, R0 + ROWS) - 1) / heads;
  int t = t_first;
  while (t <= t_last) {
    const int rq = req[t];
    int t_end = t;
    while (t_end + 1 <= t_last && req[t_end + 1] == rq) ++t_end;
    const int kv_end = pos[t_end] + 1, kv_lo = window > 0 ? max(pos[t] - window + 1, 0) : 0;  // keys any row of this run can see
    const int per = ((kv_end - kv_lo + nsplit - 1) / nsplit + kMmaKeys - 1) / kMmaKeys * kMmaKeys;
    const int k_begin = kv_lo + split * per, k_end = min(kv_end, k_begin + per);
    const int* pg = pages + page_off[rq];
    bool act[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) act[i] = row_tok[i] >= t && row_tok[i] <= t_end;

    auto load_keys = [&](int j0, int buf) {
      bf16* base = Ks + (size_t)buf * kMmaKeys * ldk;
      int r = ld_r0, c = ld_c0;  // (key row, 16-byte piece) of this thread's first piece; the next one is nthreads pieces on
      while (r < kMmaKeys) {
        const int j = j0 + r;
        bf16* dst = base + r * ldk + c * 8;
        if (j < k_end) {
          const int page = ps_shift >= 0 ? pg[j >> ps_shift] : pg[j / page_size];
          const int slot = ps_shift >= 0 ? (j & (page_size - 1)) : j % page_size;
          cp_async16(dst, cache + (size_t)page * page_stride + (size_t)slot * D + c * 8);
        } else {
          *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        r += ld_dr;
        c += ld_dc;
        if (c >= chunks) {
          c -= chunks;
          ++r;
        }
      }
      cp_async_commit();
    };

    if (k_begin < k_end) load_keys(k_begin, 0);
    int it = 0;
    for (int j0 = k_begin; j0 < k_end; j0 += kMmaKeys, ++it) {
      const int buf = it & 1;
      cp_async_wait_all();
      __syncthreads();  // tile `it` (and Q) landed; everyone is done with the other buffer, Ps and the statistics
      if (j0 + kMmaKeys < k_end) load_keys(j0 + kMmaKeys, buf ^ 1);
      const bf16* Kt = Ks + (size_t)buf * kMmaKeys * ldk;

      // ---- S = Q K^T for this warp's 16 keys, all query tiles
      float s[MT][2][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) s[mt][nt][0] = s[mt][nt][1] = s[mt][nt][2] = s[mt][nt][3] = 0.f;
      for (int kk = 0; kk < D; kk += 16) {
        uint32_t b[4];
        ldsm_x4(b, Kt + (warp * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * ldk + kk + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          uint32_t a[4];
          ldsm_x4(a, Qs + (rb + mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldk + kk + ((lane >> 4) & 1) * 8);
          mma_bf16_16816(s[mt][0], a, b[0], b[1]);
          mma_bf16_16816(s[mt][1], a, b[2], b[3]);
        }
      }
      float mx[NR];
#pragma unroll
      for (int i = 0; i < NR; ++i) mx[i] = kNegBig;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = mt * 2 + (e >> 1), j = j0 + warp * 16 + nt * 8 + 2 * tq + (e & 1);
            const bool vis = act[i] && j < k_end && j <= row_pos[i] && (window <= 0 || j > row_pos[i] - window);
            s[mt][nt][e] = vis ? s[mt][nt][e] * scale : kNegBig;
            mx[i] = fmaxf(mx[i], s[mt][nt][e]);
          }
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        if (tq == 0) wmax[warp * ROWS + rb + g + 8 * i] = mx[i];
      }
      __syncthreads();
      float corr[NR], m_new[NR], ps[NR];
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int r = rb + g + 8 * i;
        m_new[i] = fmaxf(fmaxf(fmaxf(wmax[r], wmax[ROWS + r]), fmaxf(wmax[2 * ROWS + r], wmax[3 * ROWS + r])), m_run[i]);
        corr[i] = __expf(m_run[i] - m_new[i]);
        ps[i] = 0.f;
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          float p[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = mt * 2 + (e >> 1);
            p[e] = s[mt][nt][e] <= -1e29f ? 0.f : __expf(s[mt][nt][e] - m_new[i]);
            ps[i] += p[e];
          }
          const int col = warp * 16 + nt * 8 + 2 * tq;
          *reinterpret_cast<uint32_t*>(Ps + (rb + mt * 16 + g) * 72 + col) = pack_bf16(p[0], p[1]);
          *reinterpret_cast<uint32_t*>(Ps + (rb + mt * 16 + g + 8) * 72 + col) = pack_bf16(p[2], p[3]);
        }
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], 1);
        ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], 2);
        if (tq == 0) wsum[warp * ROWS + rb + g + 8 * i] = ps[i];
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int r = rb + g + 8 * i;
        l_run[i] = l_run[i] * corr[i] + (wsum[r] + wsum[ROWS + r]) + (wsum[2 * ROWS + r] + wsum[3 * ROWS + r]);
        m_run[i] = m_new[i];
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int n = 0; n < NV; ++n) {
          o[mt][n][0] *= corr[2 * mt];
          o[mt][n][1] *= corr[2 * mt];
          o[mt][n][2] *= corr[2 * mt + 1];
          o[mt][n][3] *= corr[2 * mt + 1];
        }
      // ---- O += P V over this warp's output columns
      const int vcol0 = warp * (rank / 4);
#pragma unroll
      for (int ks = 0; ks < kMmaKeys / 16; ++ks) {
        uint32_t a[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          ldsm_x4(a[mt], Ps + (rb + mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * 72 + ks * 16 + ((lane >> 4) & 1) * 8);
#pragma unroll
        for (int np = 0; np < NV / 2; ++np) {
          if (np * 2 < nv) {
            uint32_t b[4];
            ldsm_x4_trans(b, Kt + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldk + vcol0 + np * 16 + ((lane >> 4) & 1) * 8);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              mma_bf16_16816(o[mt][2 * np], a[mt], b[0], b[1]);
              mma_bf16_16816(o[mt][2 * np + 1], a[mt], b[2], b[3]);
            }
          }
        }
      }
    }
    __syncthreads();  // the next request's first load reuses buffer 0
    t = t_end + 1;
  }
  cp_async_wait_all();  // a tile with no keys in this split still waits for its Q copy

  // ---- write: final rows (one split) or partial state (several)
  const int vcol0 = warp * (rank / 4);
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int r = rb + g + 8 * i, R = R0 + r, mt = i >> 1, hf = i & 1;
    if (R >= total_rows) continue;
    if (nsplit == 1) {
      const float sk = sink ? bf2f(sink[R % heads]) : kNegBig;
      const float M = fmaxf(m_run[i], sk);
      const float w = __expf(m_run[i] - M);
      const float inv = w / (l_run[i] * w + (sink ? __expf(sk - M) : 0.f));
#pragma unroll
      for (int n = 0; n < NV; ++n)
        if (n < nv)
          *reinterpret_cast<uint32_t*>(out + (size_t)R * rank + vcol0 + n * 8 + 2 * tq) = pack_bf16(o[mt][n][2 * hf] * inv, o[mt][n][2 * hf + 1] * inv);
    } else {
      const size_t slot = ((size_t)blockIdx.x * nsplit + split) * ROWS + r;
      if (warp == 0 && tq == 0) {
        part_ml[slot * 2] = m_run[i];
        part_ml[slot * 2 + 1] = l_run[i];
      }
#pragma unroll
      for (int n = 0; n < NV; ++n)
        if (n < nv) *reinterpret_cast<float2*>(part_o + slot * rank + vcol0 + n * 8 + 2 * tq) = make_float2(o[mt][n][2 * hf], o[mt][n][2 * hf + 1]);
    }
  }
}

// one block per query row: combine the splits' (m, l, O) and the sink
__global__ void latent_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const bf16* __restrict__ sink,
                                              bf16* __restrict__ out, int nsplit, int heads, int rank, int tile_rows) {
  __shared__ float wgt[64];  // per split: exp(m_s - M) / denominator
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int R = blockIdx.x, tile = R / tile_rows, r = R % tile_rows;
  const size_t slot0 = (size_t)tile * nsplit * tile_rows + r;  // split s at slot0 + s * tile_rows
  if (threadIdx.x < 32) {
    const float sk = sink ? bf2f(sink[R % heads]) : kNegBig;
    float m[2], l[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int s = threadIdx.x + 32 * i;
      m[i] = s < nsplit ? part_ml[(slot0 + (size_t)s * tile_rows) * 2] : kNegBig;
      l[i] = s < nsplit ? part_ml[(slot0 + (size_t)s * tile_rows) * 2 + 1] : 0.f;
    }
    const float M = fmaxf(warp_max(fmaxf(m[0], m[1])), sk);
    const float e0 = __expf(m[0] - M), e1 = __expf(m[1] - M);
    const float inv = 1.f / (warp_sum(l[0] * e0 + l[1] * e1) + (sink ? __expf(sk - M) : 0.f));
    wgt[threadIdx.x] = e0 * inv;
    wgt[threadIdx.x + 32] = e1 * inv;
  }
  __syncthreads();
  const int d = blockIdx.y * blockDim.x + threadIdx.x;  // one output column per thread; the splits' loads are independent
  if (d < rank) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int s = 0;
    for (; s + 4 <= nsplit; s += 4) {
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = part_o[(slot0 + (size_t)(s + u) * tile_rows) * rank + d];
#pragma unroll
      for (int u = 0; u < 4; ++u) acc[u] = fmaf(v[u], wgt[s + u], acc[u]);
    }
    for (; s < nsplit; ++s) acc[0] = fmaf(part_o[(slot0 + (size_t)s * tile_rows) * rank + d], wgt[s], acc[0]);
    out[(size_t)R * rank + d] = f2bf((acc[0] + acc[1]) + (acc[2] + acc[3]));
  }
}

template <int NV, int MT, int WG>
static cudaError_t launch_mma(dim3 grid, size_t smem, cudaStream_t st, const bf16* qa, const bf16* cache, const bf16* sink, const int* pos, const int* req,
                              const int* page_off, const int* pages, bf16* out, float* po, float* pml, long page_stride, int page_size, int tokens,
                              int heads, int rank, int rot, float scale, int window) {
  static bool attr_done = false;
  if (!attr_done) {
    cudaFuncSetAttribute(latent_attention_mma_kernel<NV, MT, WG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    attr_done = true;
  }
  return launch(latent_attention_mma_kernel<NV, MT, WG>, grid, dim3(128 * WG), smem, st, true, qa, cache, sink, pos, req, page_off, pages, out, po, pml,
                page_stride, page_size, tokens, heads, rank, rot, scale, window);
}

static size_t mma_smem_bytes(int rows, int D) { return (size_t)(rows + 2 * kMmaKeys) * (D + 8) * 2 + (size_t)rows * 72 * 2 + (size_t)8 * rows * 4; }

// 0 = launched; -2 = shape / alignment outside this kernel (the caller runs the generic kernel)
int launch_latent_attention_mma(const bf16* qa, const bf16* cache, const bf16* sink, const int* pos, const int* req, const int* page_off,
                                const int* pages, bf16* out, long page_stride, int page_size, int tokens, int heads, int rank, int rot, float scale,
                                int window, int max_kv_len, cudaStream_t st) {
  const int D = rank + rot;
  if (window > 0) max_kv_len = min(max_kv_len, window + tokens);  // no row sees more keys than that
  if (rank % 64 || rot % 16 || rank > 512 || page_stride % 8 || (reinterpret_cast<uintptr_t>(qa) & 15) || (reinterpret_cast<uintptr_t>(cache) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 3))
    return -2;
  if (mma_smem_bytes(16, D) > 200 * 1024) return -2;
  // 32-row CTAs (two warp groups) once there are enough rows to fill the GPU with them; 16-row CTAs, key axis split, for a decode step
  const int total = tokens * heads;
  const int wg = (total >= 32 * sm_count() && mma_smem_bytes(32, D) <= 200 * 1024) ? 2 : 1;
  const int rows = 16 * wg;
  const size_t smem = mma_smem_bytes(rows, D);
  const int tiles = (total + rows - 1) / rows;
  int splits = 1;
  ThreadState& ts = tls();
  if (max_kv_len > 2 * kMmaKeys && tiles < 2 * sm_count() && ts.scratch) {
    splits = min(min((2 * sm_count() + tiles - 1) / tiles, (max_kv_len + kMmaKeys - 1) / kMmaKeys), 64);
    while (splits > 1 && (size_t)tiles * splits * rows * (rank + 2) * 4 > ts.scratch_bytes) --splits;
  }
  float* po = static_cast<float*>(ts.scratch);
  float* pml = po ? po + (size_t)tiles * splits * rows * rank : nullptr;
  const dim3 grid(tiles, splits);
  const int nv = rank / 32;
  cudaError_t e;
#define PK_LAUNCH_MMA(NVV, WGG) \
  launch_mma<NVV, 1, WGG>(grid, smem, st, qa, cache, sink, pos, req, page_off, pages, out, po, pml, page_stride, page_size, tokens, heads, rank, rot, scale, window)
  if (wg == 2) {
    if (nv <= 2) e = PK_LAUNCH_MMA(2, 2);
    else if (nv <= 4) e = PK_LAUNCH_MMA(4, 2);
    else if (nv <= 8) e = PK_LAUNCH_MMA(8, 2);
    else e = PK_LAUNCH_MMA(16, 2);
  } else {
    if (nv <= 2) e = PK_LAUNCH_MMA(2, 1);
    else if (nv <= 4) e = PK_LAUNCH_MMA(4, 1);
    else if (nv <= 8) e = PK_LAUNCH_MMA(8, 1);
    else e = PK_LAUNCH_MMA(16, 1);
  }
#undef PK_LAUNCH_MMA
  if (e != cudaSuccess) return (int)e;
  if (splits > 1)
    e = launch(latent_attention_merge_kernel, dim3(total, (rank + 127) / 128), dim3(128), 0, st, true, (const float*)po, (const float*)pml, sink, out, splits, heads, rank,
               rows);
  return (int)e;
}

}  // namespace pk
