// Strided batched product on the tensor cores (bf16, fp32 accumulation) for the per-head factor products of the latent
// attention over many tokens: C[b][i][j] = f(row_scale[i*ld_scale + b]) * sum_k A[b*bsA + i*lda + k] * B[b*bsB + j*ldb + k].
// Both operands are contraction-major, so there are no transposes; 64 x 64 x 32 tiles, 4 warps of 32 x 32, mma.sync
// m16n8k16, operands through a two-stage cp.async ring (the tile loop of moe_grouped.cu without the row gather).
// Tensor-bound: 2 * batch * rows * cols * K flop.
#include "common.cuh"
#include "mma.cuh"

namespace pk {

constexpr int kBT = 64, kBK = 32, kBLd = kBK + 8;

template <typename OUT>  // bf16, or float for products whose result must stay fp32 (router logits, gates)
__global__ void __launch_bounds__(128) gemm_batched_mma_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B, OUT* __restrict__ C,
                                                              const float* __restrict__ row_scale, int rows, int cols, int K, long lda, long ldb,
                                                              long ldc, long bsA, long bsB, long bsC, int ld_scale, int scale_kind) {
  __shared__ __align__(16) bf16 As[2][kBT * kBLd];
  __shared__ __align__(16) bf16 Bs[2][kBT * kBLd];
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int bz = blockIdx.z, m0 = blockIdx.y * kBT, n0 = blockIdx.x * kBT;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tq = lane & 3, wm = warp >> 1, wn = warp & 1;
  A += (size_t)bz * bsA;
  B += (size_t)bz * bsB;
  C += (size_t)bz * bsC;
  const bf16* a_src[2];
  const bf16* b_src[2];
  int kc[2], sm_off[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int c = tid + i * 128, r = c >> 2;
    kc[i] = (c & 3) * 8;
    sm_off[i] = r * kBLd + kc[i];
    a_src[i] = m0 + r < rows ? A + (size_t)(m0 + r) * lda : nullptr;
    b_src[i] = n0 + r < cols ? B + (size_t)(n0 + r) * ldb : nullptr;
  }
  auto load = [&](int kt, int buf) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int k = kt * kBK + kc[i];
      if (a_src[i] && k < K) cp_async16(&As[buf][sm_off[i]], a_src[i] + k);
      else *reinterpret_cast<uint4*>(&As[buf][sm_off[i]]) = make_uint4(0, 0, 0, 0);
      if (b_src[i] && k < K) cp_async16(&Bs[buf][sm_off[i]], b_src[i] + k);
      else *reinterpret_cast<uint4*>(&Bs[buf][sm_off[i]]) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
  };
  float acc[2][4][4] = {};
  const int nk = (K + kBK - 1) / kBK;
  load(0, 0);
  for (int kt = 0; kt < nk; ++kt) {
    const int buf = kt & 1;
    cp_async_wait_all();
    __syncthreads();
    if (kt + 1 < nk) load(kt + 1, buf ^ 1);
#pragma unroll
    for (int kk = 0; kk < kBK; kk += 16) {
      uint32_t a[2][4], b[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
        ldsm_x4(a[mi], &As[buf][(wm * 32 + mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kBLd + kk + ((lane >> 4) & 1) * 8]);
#pragma unroll
      for (int np = 0; np < 2; ++np)
        ldsm_x4(b[np], &Bs[buf][(wn * 32 + np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * kBLd + kk + ((lane >> 3) & 1) * 8]);
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
      const int i = m0 + wm * 32 + mi * 16 + g + hf * 8;
      if (i >= rows) continue;
      float s = 1.f;
      if (row_scale) {
        s = row_scale[(size_t)i * ld_scale + bz];
        if (scale_kind == 2) s = 1.f / (1.f + expf(-s));
      }
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) {
        const int j = n0 + wn * 32 + ni * 8 + 2 * tq;
        OUT* o = C + (size_t)i * ldc + j;
        const float v0 = acc[mi][ni][hf * 2] * s, v1 = acc[mi][ni][hf * 2 + 1] * s;
        if constexpr (sizeof(OUT) == 4) {
          if (j < cols) o[0] = v0;
          if (j + 1 < cols) o[1] = v1;
        } else {
          if (j + 1 < cols && (reinterpret_cast<uintptr_t>(o) & 3) == 0) *reinterpret_cast<uint32_t*>(o) = pack_bf16(v0, v1);
          else {
            if (j < cols) o[0] = f2bf(v0);
            if (j + 1 < cols) o[1] = f2bf(v1);
          }
        }
      }
    }
}

// 0 = launched, -2 = operands not laid out for this kernel (the caller runs the plain FMA kernel)
int launch_gemm_batched_mma(const bf16* A, const bf16* B, bf16* C, const float* row_scale, int rows, int cols, int K, long lda, long ldb, long ldc,
                            int batch, long bsA, long bsB, long bsC, int ld_scale, int scale_kind, cudaStream_t st) {
  if (K % 8 || lda % 8 || ldb % 8 || bsA % 8 || bsB % 8 || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -2;
  const cudaError_t e = launch(gemm_batched_mma_kernel<bf16>, dim3((cols + kBT - 1) / kBT, (rows + kBT - 1) / kBT, batch), dim3(128), 0, st, true, A, B,
                               C, row_scale, rows, cols, K, lda, ldb, ldc, bsA, bsB, bsC, ld_scale, scale_kind);
  return (int)e;
}

}  // namespace pk

// out[t][m] (fp32) = W[m] . xa[t] with bf16 operands and fp32 accumulation: the skinny projections (router logits, gates) of a
// prompt portion on the tensor cores.  -2: K not a multiple of 8 or misaligned (the caller runs pk_res32_skinny_proj).
extern "C" int pk_proj_rows_f32out(const void* W, const void* xa, float* out, int M, int K, int tokens, pk_stream st) {
  using namespace pk;
  if (!W || !xa || !out || M <= 0 || K <= 0 || tokens <= 0) return -1;
  if (K % 8 || (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(xa) & 15)) return -2;
  return (int)launch(gemm_batched_mma_kernel<float>, dim3((M + kBT - 1) / kBT, (tokens + kBT - 1) / kBT, 1), dim3(128), 0, st, true, (const bf16*)xa,
                     (const bf16*)W, out, (const float*)nullptr, tokens, M, K, (long)K, (long)K, (long)M, 0L, 0L, 0L, 0, 0);
}
