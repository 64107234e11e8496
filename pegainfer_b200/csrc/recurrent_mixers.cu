// Recurrent mixers with a matrix state per head, for ragged batches whose requests keep their state in numbered slots:
//   * short causal convolution + SiLU over time per channel, with the last taps - 1 inputs of every request as state;
//   * gated delta rule:   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q        (q, k unit vectors per head)
//   * xLSTM matrix memory: m' = max(f + m, i);  S <- e^(f + m - m') S + e^(i - m') k v^T;  n likewise with k alone;
//                          o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)        (i, f soft-capped log gates, m starts at 0)
//     slot layout: S [H][dim][vdim], n [H][dim], m [H][vdim + 1] (every column keeps its own copy of the running maximum)
//   * per-head RMS norm of the read-out times a weight times an activation of a gate projection.
// State, gates, decays, unit norms and the recurrences are fp32 whatever the element type E of the activations is.
//
// Step layout: entry e of the step owns rows [row0[e], row0[e] + len[e]) of every [tokens, features] buffer (a portion
// of a prompt or one decoded token) and the state slot slot[e]; a slot's state is `state + slot * slot_stride` floats.
// Sequence kernels: one CTA per (entry, head, slice of value columns); a thread owns one column of S in registers
// (key size padded to the template's DK), tokens run one after the other, per block of kSeqTB tokens the unit keys /
// queries and the gates are prepared by all warps in shared memory.  The matrix memory's normaliser n is one more
// column with value 1.  Latency-bound per token (3 DK dependent FMAs per column, split over 4 partial sums).
#include "common.cuh"
#include "typed.cuh"

namespace pk {

constexpr int kSeqTB = 16;  // tokens prepared per block

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float logsigmoidf_(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// y[t][c] = silu(sum_j w[c][j] * x[t - (taps-1-j)][c]); inputs before this step's rows come from the slot's state
// [taps-1][C] (oldest first; zero for a new request).  in / out may have different row strides; out may alias nothing of in.
template <typename E>
__global__ void causal_conv_silu_kernel(const E* __restrict__ in, int ld_in, const E* __restrict__ w, const float* __restrict__ state, long slot_stride,
                                        const int* __restrict__ req, const int* __restrict__ slot, const int* __restrict__ row0, E* __restrict__ out,
                                        int ld_out, int C, int taps, long total) {
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int t = (int)(i / C), c = (int)(i % C), e = req[t], off = t - row0[e];
    const float* st = state + (size_t)slot[e] * slot_stride;
    float acc = 0.f;
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
  int H, G, dim, vdim, cols_per_cta;
  float cap;           // matrix memory: gate soft cap
};

// MODE 0: gated delta rule.  MODE 1: xLSTM matrix memory.
template <typename E, int DK, int MODE>
__global__ void __launch_bounds__(128) recurrent_seq_kernel(SeqArgs a) {
  __shared__ __align__(16) float ks[kSeqTB][DK];
  __shared__ __align__(16) float qs[kSeqTB][DK];
  __shared__ float g0[kSeqTB], g1[kSeqTB];  // delta: decay, beta;  memory: log forget gate, log input gate
  pdl_wait();
  pdl_launch_dependents();  // the next kernel may start its launch; it waits for this grid to finish before it reads
  const int e = blockIdx.x, h = blockIdx.y, kvh = h / (a.H / a.G);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  const int n = a.len[e], r0 = a.row0[e], dim = a.dim, vdim = a.vdim;
  const int col = blockIdx.z * a.cols_per_cta + tid;
  const int col_end = min(vdim, (int)(blockIdx.z + 1) * a.cols_per_cta);
  // the normaliser column of the matrix memory rides in the first CTA of the head, after its value columns
  const bool is_n = MODE == 1 && blockIdx.z == 0 && tid == min(a.cols_per_cta, vdim);
  const bool is_v = tid < a.cols_per_cta && col < col_end;
  float* base = a.state + (size_t)a.slot[e] * a.slot_stride;
  float* S_g = base + (size_t)h * dim * vdim;               // [dim][vdim]
  float* n_g = base + (size_t)a.H * dim * vdim + (size_t)h * dim;  // matrix memory only
  float* m_g = base + (size_t)a.H * dim * vdim + (size_t)a.H * dim + (size_t)h * (vdim + 1) + (is_v ? col : vdim);  // one copy per column: CTAs of a head never read what another one wrote
  float S[DK];
#pragma unroll
  for (int i = 0; i < DK; ++i) S[i] = (i < dim) ? (is_v ? S_g[(size_t)i * vdim + col] : (is_n ? n_g[i] : 0.f)) : 0.f;
  float m = (MODE == 1 && (is_v || is_n)) ? m_g[0] : 0.f;
  const E* X = static_cast<const E*>(a.qkv);
  const float qscale = 1.f / sqrtf((float)dim);
  for (int b0 = 0; b0 < n; b0 += kSeqTB) {
    const int nb = min(kSeqTB, n - b0);
    __syncthreads();
    for (int tt = warp; tt < nb; tt += nw) {
      const size_t row = (size_t)(r0 + b0 + tt);
      const E* qr = X + row * a.ld + a.q_off + kvh * dim;
      const E* kr = X + row * a.ld + a.k_off + kvh * dim;
      float qq = 0.f, kk = 0.f;
      for (int i = lane; i < dim; i += 32) {
        const float qv = to_f(qr[i]), kv = to_f(kr[i]);
        qq = fmaf(qv, qv, qq);
        kk = fmaf(kv, kv, kk);
      }
      float qf = qscale, kf = 1.f;
      if (MODE == 0) {
        qq = warp_sum(qq);
        kk = warp_sum(kk);
        qf = qscale / sqrtf(qq + 1e-6f);
        kf = 1.f / sqrtf(kk + 1e-6f);
      }
      for (int i = lane; i < DK; i += 32) {
        qs[tt][i] = i < dim ? to_f(qr[i]) * qf : 0.f;
        ks[tt][i] = i < dim ? to_f(kr[i]) * kf : 0.f;
      }
      if (lane == 0) {
        const float za = a.z[row * a.ldz + a.za_off + h], zb = a.z[row * a.ldz + a.zb_off + h];
        if (MODE == 0) {  // za: decay projection, zb: write-strength projection
          g0[tt] = expf(-expf(a.p0[h]) * softplusf_(za + a.p1[h]));
          g1[tt] = sigmoidf_(zb);
        } else {  // za: forget gate, zb: input gate
          g0[tt] = logsigmoidf_(a.cap * tanhf((za + a.p1[h]) / a.cap));
          g1[tt] = a.cap * tanhf((zb + a.p0[h]) / a.cap);
        }
      }
    }
    __syncthreads();
    if (!is_v && !is_n) continue;
    for (int tt = 0; tt < nb; ++tt) {
      const size_t row = (size_t)(r0 + b0 + tt);
      const float vt = is_v ? to_f(X[row * a.ld + a.v_off + h * vdim + col]) : 1.f;
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
      if (MODE == 0) {
        const float g = g0[tt], beta = g1[tt];
        float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
#pragma unroll
        for (int i = 0; i < DK; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(&ks[tt][i]);
          S[i] *= g;
          S[i + 1] *= g;
          S[i + 2] *= g;
          S[i + 3] *= g;
          c0 = fmaf(S[i], k4.x, c0);
          c1 = fmaf(S[i + 1], k4.y, c1);
          c2 = fmaf(S[i + 2], k4.z, c2);
          c3 = fmaf(S[i + 3], k4.w, c3);
        }
        const float u = beta * (vt - ((c0 + c1) + (c2 + c3)));
#pragma unroll
        for (int i = 0; i < DK; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(&ks[tt][i]);
          const float4 q4 = *reinterpret_cast<const float4*>(&qs[tt][i]);
          S[i] = fmaf(k4.x, u, S[i]);
          S[i + 1] = fmaf(k4.y, u, S[i + 1]);
          S[i + 2] = fmaf(k4.z, u, S[i + 2]);
          S[i + 3] = fmaf(k4.w, u, S[i + 3]);
          o0 = fmaf(S[i], q4.x, o0);
          o1 = fmaf(S[i + 1], q4.y, o1);
          o2 = fmaf(S[i + 2], q4.z, o2);
          o3 = fmaf(S[i + 3], q4.w, o3);
        }
        a.out[row * ((size_t)a.H * vdim) + h * vdim + col] = (o0 + o1) + (o2 + o3);
      } else {
        const float f = g0[tt], ig = g1[tt];
        const float mn = fmaxf(f + m, ig);
        const float fa = expf(f + m - mn), wb = expf(ig - mn) * vt;
        m = mn;
#pragma unroll
        for (int i = 0; i < DK; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(&ks[tt][i]);
          const float4 q4 = *reinterpret_cast<const float4*>(&qs[tt][i]);
          S[i] = fmaf(k4.x, wb, fa * S[i]);
          S[i + 1] = fmaf(k4.y, wb, fa * S[i + 1]);
          S[i + 2] = fmaf(k4.z, wb, fa * S[i + 2]);
          S[i + 3] = fmaf(k4.w, wb, fa * S[i + 3]);
          o0 = fmaf(S[i], q4.x, o0);
          o1 = fmaf(S[i + 1], q4.y, o1);
          o2 = fmaf(S[i + 2], q4.z, o2);
          o3 = fmaf(S[i + 3], q4.w, o3);
        }
        const float o = (o0 + o1) + (o2 + o3);
        if (is_v) a.out[row * ((size_t)a.H * vdim) + h * vdim + col] = o;
        else a.den[row * a.H + h] = fmaxf(fabsf(o), expf(-mn)) + 1e-6f;
      }
    }
  }
  if (is_v) {
#pragma unroll
    for (int i = 0; i < DK; ++i)
      if (i < dim) S_g[(size_t)i * vdim + col] = S[i];
    if (MODE == 1) m_g[0] = m;
  } else if (is_n) {
#pragma unroll
    for (int i = 0; i < DK; ++i)
      if (i < dim) n_g[i] = S[i];
    m_g[0] = m;
  }
}

// out[t, h, j] = E( (o[t,h,j] / den[t,h]) / sqrt(mean_j(.^2) + eps) * w[h * w_stride + j] * act(gate[t, gate_off + h*vdim + j]) )
// act 0: silu, 1: logistic.  den may be null.  One warp per (token, head).
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
    const float v = den ? orow[j] / den[pr] : orow[j];
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)vdim + eps);
  for (int j = lane; j < vdim; j += 32) {
    const float v = den ? orow[j] / den[pr] : orow[j];
    const float gz = to_f(gate[(size_t)t * ld_gate + gate_off + h * vdim + j]);
    const float ga = act == 0 ? gz / (1.f + expf(-gz)) : 1.f / (1.f + expf(-gz));
    out[pr * vdim + j] = from_f<E>(v * inv * to_f(w[(size_t)h * w_stride + j]) * ga);
  }
}

template <typename E, int MODE>
static int launch_seq(const SeqArgs& a, int entries, cudaStream_t st) {
  // columns per CTA: whole warps; short steps (decoding) spread a head over more CTAs
  int cols = a.vdim <= 32 ? a.vdim : (a.vdim + 1) / 2;
  if (cols > 96) cols = 96;
  if (cols > 32) cols = (cols + 31) / 32 * 32;
  if (cols > a.vdim) cols = a.vdim;
  SeqArgs b = a;
  b.cols_per_cta = cols;
  const int threads = std::min(128, (cols + (MODE == 1 ? 1 : 0) + 31) / 32 * 32);
  if (cols + (MODE == 1 ? 1 : 0) > threads) {  // the extra column does not fit: one warp less of value columns
    b.cols_per_cta = cols = threads - 32;
  }
  const dim3 grid(entries, a.H, (a.vdim + cols - 1) / cols);
  const int dk = a.dim <= 32 ? 32 : a.dim <= 64 ? 64 : a.dim <= 128 ? 128 : 256;
  if (a.dim > 256) return -2;
  if (dk == 32) launch(recurrent_seq_kernel<E, 32, MODE>, grid, dim3(threads), 0, st, true, b);
  else if (dk == 64) launch(recurrent_seq_kernel<E, 64, MODE>, grid, dim3(threads), 0, st, true, b);
  else if (dk == 128) launch(recurrent_seq_kernel<E, 128, MODE>, grid, dim3(threads), 0, st, true, b);
  else launch(recurrent_seq_kernel<E, 256, MODE>, grid, dim3(threads), 0, st, true, b);
  return (int)cudaGetLastError();
}

static inline int grid_for(long n, int block) { return (int)std::min<long>((n + block - 1) / block, 148L * 16); }

}  // namespace pk

using namespace pk;

extern "C" int pk_causal_conv_silu(const void* in, int ld_in, const void* w, float* state, long slot_stride, const int* req, const int* slot,
                                   const int* row0, const int* len, void* out, int ld_out, int channels, int taps, int tokens, int entries, int f32,
                                   pk_stream st) {
  if (!in || !w || !state || !req || !slot || !row0 || !len || !out || channels <= 0 || taps <= 0 || tokens <= 0 || entries <= 0) return -1;
  const long total = (long)tokens * channels;
  if (f32)
    launch(causal_conv_silu_kernel<float>, dim3(grid_for(total, 256)), dim3(256), 0, st, true, (const float*)in, ld_in, (const float*)w, (const float*)state,
           slot_stride, req, slot, row0, (float*)out, ld_out, channels, taps, total);
  else
    launch(causal_conv_silu_kernel<bf16>, dim3(grid_for(total, 256)), dim3(256), 0, st, true, (const bf16*)in, ld_in, (const bf16*)w, (const float*)state,
           slot_stride, req, slot, row0, (bf16*)out, ld_out, channels, taps, total);
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
            heads, kv_heads, dim, vdim, 0, 0.f};
  return f32 ? launch_seq<float, 0>(a, entries, st) : launch_seq<bf16, 0>(a, entries, st);
}

extern "C" int pk_mlstm_seq(const void* qkv, int ld, int q_off, int k_off, int v_off, const float* z, int ldz, int forget_off, int input_off,
                            const float* input_bias, const float* forget_bias, float cap, float* state, long slot_stride, const int* slot,
                            const int* row0, const int* len, float* out, float* den, int heads, int dim, int vdim, int entries, int f32,
                            pk_stream st) {
  if (!seq_args_ok(qkv, z, input_bias, forget_bias, state, slot, row0, len, out, heads, heads, dim, vdim, entries) || !den || !(cap > 0.f)) return -1;
  SeqArgs a{qkv, ld, q_off, k_off, v_off, z, ldz, forget_off, input_off, input_bias, forget_bias, state, slot_stride, slot, row0, len, out, den,
            heads, heads, dim, vdim, 0, cap};
  return f32 ? launch_seq<float, 1>(a, entries, st) : launch_seq<bf16, 1>(a, entries, st);
}

extern "C" int pk_head_norm_gate(const float* o, const float* den, const void* w, int w_stride, const void* gate, int ld_gate, int gate_off, void* out,
                                 int tokens, int heads, int vdim, float eps, int act, int f32, pk_stream st) {
  if (!o || !w || !gate || !out || tokens <= 0 || heads <= 0 || vdim <= 0 || act < 0 || act > 1) return -1;
  const long pairs = (long)tokens * heads;
  const dim3 g((unsigned)((pairs + 3) / 4));
  if (f32)
    launch(head_norm_gate_kernel<float>, g, dim3(128), 0, st, true, o, den, (const float*)w, w_stride, (const float*)gate, ld_gate, gate_off, (float*)out,
           heads, vdim, eps, act, pairs);
  else
    launch(head_norm_gate_kernel<bf16>, g, dim3(128), 0, st, true, o, den, (const bf16*)w, w_stride, (const bf16*)gate, ld_gate, gate_off, (bf16*)out, heads,
           vdim, eps, act, pairs);
  return (int)cudaGetLastError();
}
