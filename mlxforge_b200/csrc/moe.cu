// Mixture of experts: the router's choice and the experts' feed-forward.
//
// Router (32-bit): s = sigmoid(z) over E experts.  The experts form `n_groups` equal groups of
// neighbours; a group's score is the sum of its two largest s, and only experts of the `keep`
// best groups can be chosen (n_groups = 0: no such limit).  The `top` largest s among the
// allowed experts are chosen; their weights are s * route_scale, not renormalised.  Ties go to
// the lower index.
//
// Expert:  g = min(Wg x, limit),  u = clamp(Wu x, -limit, limit),
//          y = Wd ( g * sigmoid(alpha g) * (u + 1) )
// with the weights of all experts stacked: w_gu [E, 2, ff, H] (gate rows, then up rows) and
// w_down [E, H, ff].
//
// mf_moe_rows is the kernel for few tokens and for the 32-bit path: a block per (token, chosen
// expert) streams that expert's matrices once; the chosen experts' outputs are then added in
// the order of the choice, so a token's result does not depend on what else is in the batch.
#include "common.cuh"

__device__ __forceinline__ float moe_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

// ------------------------------------------------------------------ router
// one warp per token; dynamic shared memory per warp: s[E], sel[E], gs[n_groups]
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ z, int E, int n_groups, int keep, int top, float route_scale,
                 int* __restrict__ ids, float* __restrict__ weights, int T) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  const int per_warp = 2 * E + (n_groups > 0 ? n_groups : 1);
  float* s = sm + warp * per_warp;
  float* sel = s + E;
  float* gs = sel + E;
  for (int e = lane; e < E; e += 32) {
    s[e] = moe_sigmoid(z[(long long)t * E + e]);
    sel[e] = s[e];
  }
  __syncwarp();
  if (n_groups > 0) {
    const int per = E / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float t1 = -INFINITY, t2 = -INFINITY;
      for (int i = 0; i < per; i++) {
        const float v = s[g * per + i];
        if (v > t1) { t2 = t1; t1 = v; }
        else if (v > t2) t2 = v;
      }
      gs[g] = t1 + (t2 == -INFINITY ? 0.f : t2);
    }
    __syncwarp();
    // the `keep` best groups stay; the others' experts cannot be chosen
    for (int round = 0; round < n_groups - keep; round++) {
      float worst = INFINITY;
      int wi = -1;
      for (int g = lane; g < n_groups; g += 32) {      // the worst group, ties to the higher index
        const float v = gs[g];
        if (v <= worst && v != INFINITY) { worst = v; wi = g; }
      }
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, worst, o);
        const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
        if (oi >= 0 && (wi < 0 || ov < worst || (ov == worst && oi > wi))) { worst = ov; wi = oi; }
      }
      if (wi >= 0) {
        for (int i = lane; i < per; i += 32) sel[wi * per + i] = -INFINITY;
        if (lane == 0) gs[wi] = INFINITY;              // out of the running
      }
      __syncwarp();
    }
  }
  for (int k = 0; k < top; k++) {
    float best = -INFINITY;
    int bi = -1;
    for (int e = lane; e < E; e += 32) {
      const float v = sel[e];
      if (v > best) { best = v; bi = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
    }
    if (lane == 0) {
      ids[(long long)t * top + k] = bi < 0 ? 0 : bi;
      weights[(long long)t * top + k] = bi < 0 ? 0.f : s[bi] * route_scale;
      if (bi >= 0) sel[bi] = -INFINITY;
    }
    __syncwarp();
  }
}

MF_API int mf_moe_route(const float* z, int T, int E, int n_groups, int keep, int top, float route_scale, int* ids,
                        float* weights, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E) return MF_ERR_BAD_ARG;
  if (n_groups > 0 && (E % n_groups || keep < 1 || keep > n_groups || (long long)keep * (E / n_groups) < top))
    return MF_ERR_BAD_ARG;
  const int per_warp = 2 * E + (n_groups > 0 ? n_groups : 1);
  const size_t smem = (size_t)4 * per_warp * sizeof(float);
  if (smem > 48 * 1024) return MF_ERR_BAD_ARG;
  mf_count(MF_K_MOE_ROUTE);
  moe_route_kernel<<<(T + 3) / 4, 128, smem, stream>>>(z, E, n_groups, keep, top, route_scale, ids, weights, T);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ experts, a block per (token, choice)
// y [T, top, H] 32-bit, not yet weighted.
template <typename T>
__global__ void __launch_bounds__(256)
moe_rows_kernel(const T* __restrict__ x, const T* __restrict__ w_gu, const T* __restrict__ w_down,
                const int* __restrict__ ids, float* __restrict__ y, int H, int ff, int top, float limit, float alpha) {
  extern __shared__ float sm[];
  float* xs = sm;            // [H]
  float* act = sm + H;       // [ff]
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x, k = blockIdx.y;
  const int e = ids[(long long)t * top + k];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < H; i += blockDim.x) xs[i] = to_f32<T>(x[(long long)t * H + i]);
  __syncthreads();
  const T* wg = w_gu + (long long)e * 2 * ff * H;
  const T* wu = wg + (long long)ff * H;
  for (int f = warp; f < ff; f += nwarps) {
    const T* rg = wg + (long long)f * H;
    const T* ru = wu + (long long)f * H;
    float g = 0.f, u = 0.f;
    for (int i = lane; i < H; i += 32) {
      g = fmaf(xs[i], to_f32<T>(rg[i]), g);
      u = fmaf(xs[i], to_f32<T>(ru[i]), u);
    }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      // the activation is rounded where a product in the compute dtype would read it
      act[f] = to_f32<T>(from_f32<T>(g * moe_sigmoid(alpha * g) * (u + 1.0f)));
    }
  }
  __syncthreads();
  const T* wd = w_down + (long long)e * H * ff;
  float* yo = y + ((long long)t * top + k) * H;
  for (int c = warp; c < H; c += nwarps) {
    const T* rd = wd + (long long)c * ff;
    float a = 0.f;
    for (int i = lane; i < ff; i += 32) a = fmaf(act[i], to_f32<T>(rd[i]), a);
    a = warp_sum(a);
    if (lane == 0) yo[c] = a;
  }
}

MF_API int mf_moe_rows(const void* x, const void* w_gu, const void* w_down, int dtype, const int* ids, float* y, int T,
                       int H, int ff, int top, float limit, float alpha, cudaStream_t stream) {
  if (T <= 0) return 0;
  const size_t smem = (size_t)(H + ff) * sizeof(float);
  if (smem > 200 * 1024 || top > 65535) return MF_ERR_BAD_ARG;
  mf_count(MF_K_MOE_ROWS);
#define MR_LAUNCH(TT)                                                                                              \
  do {                                                                                                             \
    if (smem > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(moe_rows_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                           (int)smem);                                                             \
      if (e != cudaSuccess) return (int)e;                                                                         \
    }                                                                                                              \
    return (int)launch_dep(moe_rows_kernel<TT>, dim3(T, top), dim3(256), smem, stream, (const TT*)x,               \
                           (const TT*)w_gu, (const TT*)w_down, ids, y, H, ff, top, limit, alpha);                  \
  } while (0)
  if (dtype == MF_F32) MR_LAUNCH(float);
  if (dtype == MF_BF16) MR_LAUNCH(__nv_bfloat16);
#undef MR_LAUNCH
  return MF_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ the weighted sum of the chosen experts
// out[t] = sum_k weights[t, k] * y[src(t, k)], k in the order of the choice.  `slot_of` null:
// src(t, k) = t * top + k; else the row of y that holds the pair (tokens sorted by expert).
template <typename TO>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ weights, const int* __restrict__ slot_of,
                   TO* __restrict__ out, int H, int top) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; k++) {
      const long long row = slot_of ? slot_of[(long long)t * top + k] : (long long)t * top + k;
      a = fmaf(weights[(long long)t * top + k], y[row * H + i], a);
    }
    out[(long long)t * H + i] = from_f32<TO>(a);
  }
}

MF_API int mf_moe_combine(const float* y, const float* weights, const int* slot_of, void* out, int out_dtype, int T,
                          int H, int top, cudaStream_t stream) {
  if (T <= 0) return 0;
  mf_count(MF_K_MOE_COMBINE);
  if (out_dtype == MF_F32)
    return (int)launch_dep(moe_combine_kernel<float>, dim3(T), dim3(256), 0, stream, y, weights, slot_of, (float*)out,
                           H, top);
  if (out_dtype == MF_BF16)
    return (int)launch_dep(moe_combine_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, y, weights, slot_of,
                           (__nv_bfloat16*)out, H, top);
  return MF_ERR_BAD_DTYPE;
}
