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

constexpr int kMmaRows = 16, kMmaKeys = 64, kMmaThreads = 128;
constexpr float kNegBig = -1e30f;

// NV = 8-column output tiles per warp (rank = 32 * nv with nv <= NV, nv even)
template <int NV>
__global__ void __launch_bounds__(kMmaThreads)
latent_attention_mma_kernel(const bf16* __restrict__ qa, const bf16* __restrict__ cache, const bf16* __restrict__ sink, const int* __restrict__ pos,
                            const int* __restrict__ req, const int* __restrict__ page_off, const int* __restrict__ pages, bf16* __restrict__ out,
                            float* __restrict__ part_o, float* __restrict__ part_ml, long page_stride, int page_size, int tokens, int heads, int rank,
                            int rot, float scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = rank + rot, ldk = D + 8, nv = rank / 32;
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);   // [16][ldk]
  bf16* Ks = Qs + kMmaRows * ldk;                 // [2][64][ldk]
  bf16* Ps = Ks + 2 * kMmaKeys * ldk;             // [16][72]
  float* wmax = reinterpret_cast<float*>(Ps + kMmaRows * 72);  // [4][16]
  float* wsum = wmax + 64;                                     // [4][16]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tq = lane & 3;
  const int total_rows = tokens * heads, R0 = blockIdx.x * kMmaRows;
  const int split = blockIdx.y, nsplit = gridDim.y;
  pdl_wait();

  // ---- Q tile (rows past the end are zero)
  const int chunks = D / 8;  // 16-byte pieces per row
  for (int e = tid; e < kMmaRows * chunks; e += kMmaThreads) {
    const int r = e / chunks, c = e % chunks;
    bf16* dst = Qs + r * ldk + c * 8;
    if (R0 + r < total_rows) cp_async16(dst, qa + (size_t)(R0 + r) * D + c * 8);
    else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
  }
  cp_async_commit();

  // the two rows this thread owns in every accumulator: g and g + 8
  int row_tok[2], row_pos[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int R = R0 + g + 8 * i;
    row_tok[i] = R < total_rows ? R / heads : -1;
    row_pos[i] = row_tok[i] >= 0 ? pos[row_tok[i]] : -1;
  }
  float m_run[2] = {kNegBig, kNegBig}, l_run[2] = {0.f, 0.f};
  float o[NV][4];
#pragma unroll
  for (int i = 0; i < NV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  const int t_first = R0 / heads, t_last = (min(total_rows, R0 + kMmaRows) - 1) / heads;
  int t = t_first;
  while (t <= t_last) {
    const int rq = req[t];
    int t_end = t;
    while (t_end + 1 <= t_last && req[t_end + 1] == rq) ++t_end;
    const int kv_end = pos[t_end] + 1;
    const int per = ((kv_end + nsplit - 1) / nsplit + kMmaKeys - 1) / kMmaKeys * kMmaKeys;
    const int k_begin = split * per, k_end = min(kv_end, k_begin + per);
    const int* pg = pages + page_off[rq];
    bool act[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) act[i] = row_tok[i] >= t && row_tok[i] <= t_end;

    auto load_keys = [&](int j0, int buf) {
      bf16* base = Ks + (size_t)buf * kMmaKeys * ldk;
      for (int e = tid; e < kMmaKeys * chunks; e += kMmaThreads) {
        const int r = e / chunks, c = e % chunks, j = j0 + r;
        bf16* dst = base + r * ldk + c * 8;
        if (j < k_end) cp_async16(dst, cache + (size_t)pg[j / page_size] * page_stride + (size_t)(j % page_size) * D + c * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
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

      // ---- S = Q K^T for this warp's 16 keys
      float s[2][4] = {};
      for (int kk = 0; kk < D; kk += 16) {
        uint32_t a[4], b[4];
        ldsm_x4(a, Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * ldk + kk + ((lane >> 4) & 1) * 8);
        ldsm_x4(b, Kt + (warp * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * ldk + kk + ((lane >> 3) & 1) * 8);
        mma_bf16_16816(s[0], a, b[0], b[1]);
        mma_bf16_16816(s[1], a, b[2], b[3]);
      }
      float mx[2] = {kNegBig, kNegBig};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1, j = j0 + warp * 16 + nt * 8 + 2 * tq + (e & 1);
          const bool vis = act[i] && j < k_end && j <= row_pos[i];
          s[nt][e] = vis ? s[nt][e] * scale : kNegBig;
          mx[i] = fmaxf(mx[i], s[nt][e]);
        }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        if (tq == 0) wmax[warp * 16 + g + 8 * i] = mx[i];
      }
      __syncthreads();
      float corr[2], m_new[2], ps[2] = {0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = g + 8 * i;
        m_new[i] = fmaxf(fmaxf(fmaxf(wmax[r], wmax[16 + r]), fmaxf(wmax[32 + r], wmax[48 + r])), m_run[i]);
        corr[i] = __expf(m_run[i] - m_new[i]);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        float p[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1;
          p[e] = s[nt][e] <= -1e29f ? 0.f : __expf(s[nt][e] - m_new[i]);
          ps[i] += p[e];
        }
        const int col = warp * 16 + nt * 8 + 2 * tq;
        *reinterpret_cast<uint32_t*>(Ps + g * 72 + col) = pack_bf16(p[0], p[1]);
        *reinterpret_cast<uint32_t*>(Ps + (g + 8) * 72 + col) = pack_bf16(p[2], p[3]);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], 1);
        ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], 2);
        if (tq == 0) wsum[warp * 16 + g + 8 * i] = ps[i];
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = g + 8 * i;
        l_run[i] = l_run[i] * corr[i] + (wsum[r] + wsum[16 + r]) + (wsum[32 + r] + wsum[48 + r]);
        m_run[i] = m_new[i];
      }
#pragma unroll
      for (int n = 0; n < NV; ++n) {
        o[n][0] *= corr[0];
        o[n][1] *= corr[0];
        o[n][2] *= corr[1];
        o[n][3] *= corr[1];
      }
      // ---- O += P V over this warp's output columns
      const int vcol0 = warp * (rank / 4);
#pragma unroll
      for (int ks = 0; ks < kMmaKeys / 16; ++ks) {
        uint32_t a[4];
        ldsm_x4(a, Ps + ((lane & 7) + ((lane >> 3) & 1) * 8) * 72 + ks * 16 + ((lane >> 4) & 1) * 8);
#pragma unroll
        for (int np = 0; np < NV / 2; ++np) {
          if (np * 2 < nv) {
            uint32_t b[4];
            ldsm_x4_trans(b, Kt + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldk + vcol0 + np * 16 + ((lane >> 4) & 1) * 8);
            mma_bf16_16816(o[2 * np], a, b[0], b[1]);
            mma_bf16_16816(o[2 * np + 1], a, b[2], b[3]);
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
  for (int i = 0; i < 2; ++i) {
    const int r = g + 8 * i, R = R0 + r;
    if (R >= total_rows) continue;
    if (nsplit == 1) {
      const float sk = bf2f(sink[R % heads]);
      const float M = fmaxf(m_run[i], sk);
      const float w = __expf(m_run[i] - M);
      const float inv = w / (l_run[i] * w + __expf(sk - M));
#pragma unroll
      for (int n = 0; n < NV; ++n)
        if (n < nv)
          *reinterpret_cast<uint32_t*>(out + (size_t)R * rank + vcol0 + n * 8 + 2 * tq) = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
    } else {
      const size_t slot = ((size_t)blockIdx.x * nsplit + split) * kMmaRows + r;
      if (warp == 0 && tq == 0) {
        part_ml[slot * 2] = m_run[i];
        part_ml[slot * 2 + 1] = l_run[i];
      }
#pragma unroll
      for (int n = 0; n < NV; ++n)
        if (n < nv) *reinterpret_cast<float2*>(part_o + slot * rank + vcol0 + n * 8 + 2 * tq) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
    }
  }
}

// one block per query row: combine the splits' (m, l, O) and the sink
__global__ void latent_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const bf16* __restrict__ sink,
                                              bf16* __restrict__ out, int nsplit, int heads, int rank) {
  pdl_wait();
  const int R = blockIdx.x, tile = R / kMmaRows, r = R % kMmaRows;
  const float sk = bf2f(sink[R % heads]);
  float M = sk;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_ml[(((size_t)tile * nsplit + s) * kMmaRows + r) * 2]);
  float den = __expf(sk - M);
  for (int s = 0; s < nsplit; ++s) {
    const size_t slot = ((size_t)tile * nsplit + s) * kMmaRows + r;
    den += part_ml[slot * 2 + 1] * __expf(part_ml[slot * 2] - M);
  }
  const float inv = 1.f / den;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const size_t slot = ((size_t)tile * nsplit + s) * kMmaRows + r;
      acc += part_o[slot * rank + d] * __expf(part_ml[slot * 2] - M);
    }
    out[(size_t)R * rank + d] = f2bf(acc * inv);
  }
}

template <int NV>
static cudaError_t launch_mma(dim3 grid, size_t smem, cudaStream_t st, const bf16* qa, const bf16* cache, const bf16* sink, const int* pos, const int* req,
                              const int* page_off, const int* pages, bf16* out, float* po, float* pml, long page_stride, int page_size, int tokens,
                              int heads, int rank, int rot, float scale) {
  static bool attr_done = false;
  if (!attr_done) {
    cudaFuncSetAttribute(latent_attention_mma_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    attr_done = true;
  }
  return launch(latent_attention_mma_kernel<NV>, grid, dim3(kMmaThreads), smem, st, true, qa, cache, sink, pos, req, page_off, pages, out, po, pml,
                page_stride, page_size, tokens, heads, rank, rot, scale);
}

// 0 = launched; -2 = shape / alignment outside this kernel (the caller runs the generic kernel)
int launch_latent_attention_mma(const bf16* qa, const bf16* cache, const bf16* sink, const int* pos, const int* req, const int* page_off,
                                const int* pages, bf16* out, long page_stride, int page_size, int tokens, int heads, int rank, int rot, float scale,
                                int max_kv_len, cudaStream_t st) {
  const int D = rank + rot;
  if (rank % 64 || rot % 16 || rank > 512 || page_stride % 8 || (reinterpret_cast<uintptr_t>(qa) & 15) || (reinterpret_cast<uintptr_t>(cache) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 3))
    return -2;
  const size_t smem = (size_t)(kMmaRows + 2 * kMmaKeys) * (D + 8) * 2 + kMmaRows * 72 * 2 + 128 * 4;
  if (smem > 200 * 1024) return -2;
  const int tiles = (tokens * heads + kMmaRows - 1) / kMmaRows;
  int splits = 1;
  ThreadState& ts = tls();
  if (max_kv_len > 2 * kMmaKeys && tiles < 2 * sm_count() && ts.scratch) {
    splits = min(min((2 * sm_count() + tiles - 1) / tiles, (max_kv_len + 2 * kMmaKeys - 1) / (2 * kMmaKeys)), 64);
    while (splits > 1 && (size_t)tiles * splits * kMmaRows * (rank + 2) * 4 > ts.scratch_bytes) --splits;
  }
  float* po = static_cast<float*>(ts.scratch);
  float* pml = po ? po + (size_t)tiles * splits * kMmaRows * rank : nullptr;
  const dim3 grid(tiles, splits);
  const int nv = rank / 32;
  cudaError_t e;
  if (nv <= 2) e = launch_mma<2>(grid, smem, st, qa, cache, sink, pos, req, page_off, pages, out, po, pml, page_stride, page_size, tokens, heads, rank, rot, scale);
  else if (nv <= 4) e = launch_mma<4>(grid, smem, st, qa, cache, sink, pos, req, page_off, pages, out, po, pml, page_stride, page_size, tokens, heads, rank, rot, scale);
  else if (nv <= 8) e = launch_mma<8>(grid, smem, st, qa, cache, sink, pos, req, page_off, pages, out, po, pml, page_stride, page_size, tokens, heads, rank, rot, scale);
  else e = launch_mma<16>(grid, smem, st, qa, cache, sink, pos, req, page_off, pages, out, po, pml, page_stride, page_size, tokens, heads, rank, rot, scale);
  if (e != cudaSuccess) return (int)e;
  if (splits > 1)
    e = launch(latent_attention_merge_kernel, dim3(tokens * heads), dim3(128), 0, st, true, (const float*)po, (const float*)pml, sink, out, splits, heads,
               rank);
  return (int)e;
}

}  // namespace pk
