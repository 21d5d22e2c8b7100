// Several residual streams ("hyper-connections") and the kernels at their two ends.
//
// A model with S streams keeps x_1..x_S per token, [T, S, H] in 32-bit.  A sublayer reads
// u = sum_s in[s] x_s, runs on norm(u), and its result y is written back as
//   x_t <- sum_s mix[s, t] x_s + out[t] * y          (all t at once, from the old x_s).
// As with the single stream, the write-back of one sublayer is fused with the read and the
// norm of the next: one kernel applies the pending (y, mix, out) of the sublayer before,
// stores the streams, reads them with `in` and normalises.  S = 1 with mix = out = in = 1 is
// the ordinary residual sum.
//
// The norm is an RMS norm in groups: the H channels are cut into G equal consecutive groups,
// each divided by its own sqrt(mean(x^2) + eps), the whole multiplied by w.  G = 1 is RMSNorm.
//
// mf_embed_positions: token embedding plus a sinusoidal position vector (channel 2i:
// sin(p f_i), channel 2i+1: cos(p f_i), f_i = theta^(-2i/H)), written to all S streams.
// Everything here is 32-bit arithmetic; with `precise` the angle and its sine are double.
#include "common.cuh"

#define HS_MAX_STREAMS 8
#define HS_MAX_GROUPS 64
#define HS_THREADS 256

template <typename T>
__global__ void __launch_bounds__(HS_THREADS)
embed_positions_kernel(const T* __restrict__ table, const int* __restrict__ tokens, const int* __restrict__ positions,
                       const double* __restrict__ freqs, float* __restrict__ out, int H, int copies, int precise) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  const T* row = table + (long long)tokens[t] * H;
  const int p = positions[t];
  float* o = out + (long long)t * copies * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float pe = 0.f;
    if (freqs) {
      if (precise) {
        const double a = (double)p * freqs[i >> 1];
        pe = (float)((i & 1) ? cos(a) : sin(a));
      } else {
        const float a = (float)p * (float)freqs[i >> 1];
        pe = (i & 1) ? cosf(a) : sinf(a);
      }
    }
    const float v = to_f32<T>(row[i]) + pe;
    for (int c = 0; c < copies; c++) o[(long long)c * H + i] = v;
  }
}

MF_API int mf_embed_positions(const void* table, int table_dtype, const int* tokens, const int* positions,
                              const double* freqs, float* out, int T, int H, int copies, int precise,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  if (copies < 1 || H <= 0) return MF_ERR_BAD_ARG;
  mf_count(MF_K_EMBED_POSITIONS);
  if (table_dtype == MF_F32)
    return (int)launch_dep(embed_positions_kernel<float>, dim3(T), dim3(HS_THREADS), 0, stream, (const float*)table,
                           tokens, positions, freqs, out, H, copies, precise);
  if (table_dtype == MF_BF16)
    return (int)launch_dep(embed_positions_kernel<__nv_bfloat16>, dim3(T), dim3(HS_THREADS), 0, stream,
                           (const __nv_bfloat16*)table, tokens, positions, freqs, out, H, copies, precise);
  return MF_ERR_BAD_DTYPE;
}

// One block per produced row.  Without `rows` the updated streams are stored (the streams move
// on); with `rows` only the selected rows are produced and the streams are left alone.
// `delta` may be null (nothing pending); `mix`/`wout` null with a delta mean the identity and
// ones (the single residual sum); `win` null means ones (the plain sum of the streams).
template <typename TD, typename TO>
__global__ void __launch_bounds__(HS_THREADS)
hyper_update_norm_kernel(float* __restrict__ streams, const TD* __restrict__ delta,
                         const float* __restrict__ delta_bias, const float* __restrict__ mix,
                         const float* __restrict__ wout, const float* __restrict__ win,
                         const float* __restrict__ w, float eps, int groups, TO* __restrict__ out,
                         const int* __restrict__ rows, int H, int S) {
  extern __shared__ float u[];      // [H]
  __shared__ float red[32];
  __shared__ float cm[HS_MAX_STREAMS * HS_MAX_STREAMS], co[HS_MAX_STREAMS], ci[HS_MAX_STREAMS];
  __shared__ float ginv[HS_MAX_GROUPS];
  pdl_launch();
  // the stream weights never change: fetched before the wait
  if (threadIdx.x < S * S) cm[threadIdx.x] = mix ? mix[threadIdx.x] : ((threadIdx.x / S == threadIdx.x % S) ? 1.f : 0.f);
  if (threadIdx.x < S) {
    co[threadIdx.x] = wout ? wout[threadIdx.x] : 1.f;
    ci[threadIdx.x] = win ? win[threadIdx.x] : 1.f;
  }
  pdl_wait();
  __syncthreads();
  const int r = blockIdx.x;
  const long long src = rows ? rows[r] : r;
  float* x = streams + src * S * H;
  const TD* d = delta ? delta + src * H : nullptr;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float xs[HS_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HS_MAX_STREAMS; s++) xs[s] = (s < S) ? x[(long long)s * H + i] : 0.f;
    if (d) {
      const float y = to_f32<TD>(d[i]) + (delta_bias ? delta_bias[i] : 0.f);
      float nx[HS_MAX_STREAMS];
#pragma unroll
      for (int t = 0; t < HS_MAX_STREAMS; t++) {
        float a = 0.f;
        if (t < S) {
#pragma unroll
          for (int s = 0; s < HS_MAX_STREAMS; s++)
            if (s < S) a = fmaf(cm[s * S + t], xs[s], a);
          a = fmaf(co[t], y, a);
          if (!rows) x[(long long)t * H + i] = a;
        }
        nx[t] = a;
      }
#pragma unroll
      for (int s = 0; s < HS_MAX_STREAMS; s++) xs[s] = nx[s];
    }
    float a = 0.f;
#pragma unroll
    for (int s = 0; s < HS_MAX_STREAMS; s++)
      if (s < S) a = fmaf(ci[s], xs[s], a);
    u[i] = a;
  }
  __syncthreads();
  const int gs = H / groups;
  for (int g = 0; g < groups; g++) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
      const float v = u[g * gs + i];
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) ginv[g] = 1.0f / sqrtf(ss / (float)gs + eps);
  }
  __syncthreads();
  TO* o = out + (long long)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<TO>(u[i] * ginv[i / gs] * w[i]);
}

// The same with the channels in groups of four (H and the group size multiples of 4): 16-byte
// accesses to the streams, and each thread keeps its values of u in registers between the passes.
template <typename TD, typename TO, int NV>
__global__ void __launch_bounds__(HS_THREADS)
hyper_update_norm_vec_kernel(float* __restrict__ streams, const TD* __restrict__ delta,
                             const float* __restrict__ delta_bias, const float* __restrict__ mix,
                             const float* __restrict__ wout, const float* __restrict__ win,
                             const float* __restrict__ w, float eps, int groups, TO* __restrict__ out,
                             const int* __restrict__ rows, int H, int S) {
  __shared__ float red[32];
  __shared__ float cm[HS_MAX_STREAMS * HS_MAX_STREAMS], co[HS_MAX_STREAMS], ci[HS_MAX_STREAMS];
  __shared__ float gsum[HS_MAX_GROUPS];
  pdl_launch();
  if (threadIdx.x < S * S) cm[threadIdx.x] = mix ? mix[threadIdx.x] : ((threadIdx.x / S == threadIdx.x % S) ? 1.f : 0.f);
  if (threadIdx.x < S) {
    co[threadIdx.x] = wout ? wout[threadIdx.x] : 1.f;
    ci[threadIdx.x] = win ? win[threadIdx.x] : 1.f;
  }
  if (threadIdx.x < groups) gsum[threadIdx.x] = 0.f;
  pdl_wait();
  __syncthreads();
  const int r = blockIdx.x;
  const long long src = rows ? rows[r] : r;
  float* x = streams + src * S * H;
  const TD* d = delta ? delta + src * H : nullptr;
  const int gs = H / groups;
  float u[NV][4];
#pragma unroll
  for (int j = 0; j < NV; j++) {
    const int i = (j * HS_THREADS + threadIdx.x) * 4;
    u[j][0] = u[j][1] = u[j][2] = u[j][3] = 0.f;
    if (i < H) {
      float xs[HS_MAX_STREAMS][4];
#pragma unroll
      for (int s = 0; s < HS_MAX_STREAMS; s++) {
        if (s < S) {
          const float4 v = *reinterpret_cast<const float4*>(x + (long long)s * H + i);
          xs[s][0] = v.x; xs[s][1] = v.y; xs[s][2] = v.z; xs[s][3] = v.w;
        }
      }
      if (d) {
        float y[4];
#pragma unroll
        for (int e = 0; e < 4; e++) y[e] = to_f32<TD>(d[i + e]) + (delta_bias ? delta_bias[i + e] : 0.f);
        float nx[HS_MAX_STREAMS][4];
#pragma unroll
        for (int t = 0; t < HS_MAX_STREAMS; t++) {
          if (t < S) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
              float a = 0.f;
#pragma unroll
              for (int s = 0; s < HS_MAX_STREAMS; s++)
                if (s < S) a = fmaf(cm[s * S + t], xs[s][e], a);
              nx[t][e] = fmaf(co[t], y[e], a);
            }
            if (!rows)
              *reinterpret_cast<float4*>(x + (long long)t * H + i) = make_float4(nx[t][0], nx[t][1], nx[t][2], nx[t][3]);
          }
        }
#pragma unroll
        for (int s = 0; s < HS_MAX_STREAMS; s++)
          if (s < S) { xs[s][0] = nx[s][0]; xs[s][1] = nx[s][1]; xs[s][2] = nx[s][2]; xs[s][3] = nx[s][3]; }
      }
#pragma unroll
      for (int e = 0; e < 4; e++) {
        float a = 0.f;
#pragma unroll
        for (int s = 0; s < HS_MAX_STREAMS; s++)
          if (s < S) a = fmaf(ci[s], xs[s][e], a);
        u[j][e] = a;
      }
    }
  }
  // sums of squares per group, in a fixed order: group by group, each a block-wide sum
  for (int g = 0; g < groups; g++) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; j++) {
      const int i = (j * HS_THREADS + threadIdx.x) * 4;
      if (i < H && i / gs == g) ss += u[j][0] * u[j][0] + u[j][1] * u[j][1] + u[j][2] * u[j][2] + u[j][3] * u[j][3];
    }
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) gsum[g] = 1.0f / sqrtf(ss / (float)gs + eps);
  }
  __syncthreads();
  TO* o = out + (long long)r * H;
#pragma unroll
  for (int j = 0; j < NV; j++) {
    const int i = (j * HS_THREADS + threadIdx.x) * 4;
    if (i < H) {
      const float inv = gsum[i / gs];
      const float4 wv = *reinterpret_cast<const float4*>(w + i);
      o[i] = from_f32<TO>(u[j][0] * inv * wv.x);
      o[i + 1] = from_f32<TO>(u[j][1] * inv * wv.y);
      o[i + 2] = from_f32<TO>(u[j][2] * inv * wv.z);
      o[i + 3] = from_f32<TO>(u[j][3] * inv * wv.w);
    }
  }
}

MF_API int mf_hyper_update_norm(float* streams, const void* delta, int delta_dtype, const float* delta_bias,
                                const float* mix, const float* wout, const float* win, const float* w, float eps,
                                int groups, void* out, int out_dtype, const int* rows, int n, int H, int S,
                                cudaStream_t stream) {
  if (n <= 0) return 0;
  if (S < 1 || S > HS_MAX_STREAMS || groups < 1 || groups > HS_MAX_GROUPS || H % groups) return MF_ERR_BAD_ARG;
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return MF_ERR_BAD_ARG;
  mf_count(MF_K_HYPER_NORM);
#define HS_LAUNCH(TD, TO)                                                                                        \
  do {                                                                                                           \
    const bool vec = H % 4 == 0 && (H / groups) % 4 == 0 && H <= 4 * HS_THREADS * 8 &&                           \
                     ((uintptr_t)streams & 15) == 0 && ((uintptr_t)w & 15) == 0;                                 \
    if (vec && H <= 4 * HS_THREADS * 2)                                                                          \
      return (int)launch_dep(hyper_update_norm_vec_kernel<TD, TO, 2>, dim3(n), dim3(HS_THREADS), 0, stream,      \
                             streams, (const TD*)delta, delta_bias, mix, wout, win, w, eps, groups, (TO*)out,    \
                             rows, H, S);                                                                        \
    if (vec)                                                                                                     \
      return (int)launch_dep(hyper_update_norm_vec_kernel<TD, TO, 8>, dim3(n), dim3(HS_THREADS), 0, stream,      \
                             streams, (const TD*)delta, delta_bias, mix, wout, win, w, eps, groups, (TO*)out,    \
                             rows, H, S);                                                                        \
    if (smem > 48 * 1024) {                                                                                      \
      cudaError_t e = cudaFuncSetAttribute(hyper_update_norm_kernel<TD, TO>,                                     \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
      if (e != cudaSuccess) return (int)e;                                                                       \
    }                                                                                                            \
    return (int)launch_dep(hyper_update_norm_kernel<TD, TO>, dim3(n), dim3(HS_THREADS), smem, stream, streams,   \
                           (const TD*)delta, delta_bias, mix, wout, win, w, eps, groups, (TO*)out, rows, H, S);  \
  } while (0)
  if (delta_dtype == MF_F32 && out_dtype == MF_F32) HS_LAUNCH(float, float);
  if (delta_dtype == MF_BF16 && out_dtype == MF_BF16) HS_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  if (delta_dtype == MF_F32 && out_dtype == MF_BF16) HS_LAUNCH(float, __nv_bfloat16);
#undef HS_LAUNCH
  return MF_ERR_BAD_DTYPE;
}
