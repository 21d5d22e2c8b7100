// Attention whose heads talk to each other before the softmax, over the paged cache.
//
//   s_h(i, j)  = q_h(i) . k_g(h)(j) * scale
//   s_h       <- cap * tanh(s_h / cap)                      (cap > 0)
//   s'_h(i, j) = sum_g talk[h, g] * s_g(i, j)               (talk given; all heads of one query and key)
//   p_h        = softmax_j s'_h(i, j) over the keys j the query may see
//   o_h(i)     = sum_j p_h(i, j) v_g(h)(j)
//
// Keys have `dim` channels, values `vdim` (the two pools differ in their last extent).  The
// query at position i sees j <= i, further limited by a sliding window (j > i - window) and/or
// to its own chunk (floor(j / chunk) == floor(i / chunk)); chunks count from position 0 of the
// sequence.  Because the mixing couples all heads of a query, one block owns a query token
// with all its heads.  Scores, the mixing, the softmax and the sums over keys are 32-bit.
//
// Two kernels.  `talking_attention_kernel` (any dtype, any sizes): keys in tiles of 32 that
// start at multiples of 32, online softmax; it is the 32-bit path's attention and the device
// reference of the faster one.  The order of every sum depends on positions only, never on how
// a prompt was cut or what else is in the batch.
//
// mf_biased_kv_store adds the projections' biases (in 32-bit) to the step's queries, keys and
// values, rounds once, and writes keys and values into their pages.
#include "common.cuh"

#define TA_KT 32
#define TA_THREADS 256
#define TA_MAX_ACC 32

__device__ __forceinline__ long long ta_page_base(const int* block_table, int bt_stride, int page_size, int seq,
                                                  int pos, int* slot) {
  const int blk = pos / page_size;
  *slot = pos - blk * page_size;
  return block_table[(long long)seq * bt_stride + blk];
}

template <typename T>
__global__ void __launch_bounds__(TA_THREADS)
talking_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                         T* __restrict__ out, const int* __restrict__ positions,
                         const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int bt_stride,
                         int page_size, int n_heads, int n_kv, int dim, int vdim, float scale, float softcap,
                         const float* __restrict__ talk, int window, int chunk) {
  extern __shared__ float smem[];
  float* qs = smem;                          // [H * dim]
  float* sraw = qs + n_heads * dim;          // [H * KT]
  float* smix = sraw + n_heads * TA_KT;      // [H * KT]
  float* tk = smix + n_heads * TA_KT;        // [H * H]
  float* m_s = tk + n_heads * n_heads;       // [H]
  float* l_s = m_s + n_heads;                // [H]
  float* a_s = l_s + n_heads;                // [H]
  __shared__ int page_s[TA_KT], slot_s[TA_KT];
  const int t = blockIdx.x;
  const int rep = n_heads / n_kv;
  const int pos = positions[t], seq = seq_of_token[t];
  int lo = 0;
  if (window > 0 && pos - window + 1 > lo) lo = pos - window + 1;
  if (chunk > 0 && (pos / chunk) * chunk > lo) lo = (pos / chunk) * chunk;

  const T* qrow = q + (long long)t * n_heads * dim;
  for (int i = threadIdx.x; i < n_heads * dim; i += blockDim.x) qs[i] = to_f32<T>(qrow[i]);
  for (int i = threadIdx.x; i < n_heads * n_heads; i += blockDim.x)
    tk[i] = talk ? talk[i] : ((i / n_heads == i % n_heads) ? 1.f : 0.f);
  for (int i = threadIdx.x; i < n_heads; i += blockDim.x) {
    m_s[i] = -INFINITY;
    l_s[i] = 0.f;
  }
  float acc[TA_MAX_ACC];
#pragma unroll
  for (int i = 0; i < TA_MAX_ACC; i++) acc[i] = 0.f;
  const int n_out = n_heads * vdim;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  __syncthreads();

  for (int c0 = (lo / TA_KT) * TA_KT; c0 <= pos; c0 += TA_KT) {
    if (threadIdx.x < TA_KT) {
      const int pj = c0 + threadIdx.x;
      int slot = 0;
      long long page = -1;
      if (pj >= lo && pj <= pos) page = ta_page_base(block_table, bt_stride, page_size, seq, pj, &slot);
      page_s[threadIdx.x] = (int)page;
      slot_s[threadIdx.x] = slot;
    }
    __syncthreads();
    // raw scores of every (kv head, key) pair, for the query heads of that kv head
    for (int it = threadIdx.x; it < n_kv * TA_KT; it += blockDim.x) {
      const int g = it / TA_KT, j = it - g * TA_KT;
      const int page = page_s[j];
      if (page >= 0) {
        const T* kr = k_pool + (((long long)page * n_kv + g) * page_size + slot_s[j]) * dim;
        for (int r = 0; r < rep; r++) {
          const float* qh = qs + (g * rep + r) * dim;
          float dot = 0.f;
          for (int d = 0; d < dim; d++) dot = fmaf(qh[d], to_f32<T>(kr[d]), dot);
          float s = dot * scale;
          if (softcap > 0.f) s = softcap * tanhf(s / softcap);
          sraw[(g * rep + r) * TA_KT + j] = s;
        }
      } else {
        for (int r = 0; r < rep; r++) sraw[(g * rep + r) * TA_KT + j] = 0.f;
      }
    }
    __syncthreads();
    // the heads' scores mixed; a key that is not seen stays out of every head
    for (int it = threadIdx.x; it < n_heads * TA_KT; it += blockDim.x) {
      const int h = it / TA_KT, j = it - h * TA_KT;
      float s = -INFINITY;
      if (page_s[j] >= 0) {
        if (talk) {
          s = 0.f;
          for (int g = 0; g < n_heads; g++) s = fmaf(tk[h * n_heads + g], sraw[g * TA_KT + j], s);
        } else {
          s = sraw[it];
        }
      }
      smix[it] = s;
    }
    __syncthreads();
    // online softmax, a warp per head, a key per lane
    for (int h = warp; h < n_heads; h += nwarps) {
      const float s = smix[h * TA_KT + lane];
      const float cm = warp_max(s);
      const float m_old = m_s[h];
      const float m_new = fmaxf(m_old, cm);
      const float alpha = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
      const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
      const float psum = warp_sum(p);
      smix[h * TA_KT + lane] = p;
      if (lane == 0) {
        m_s[h] = m_new;
        l_s[h] = l_s[h] * alpha + psum;
        a_s[h] = alpha;
      }
    }
    __syncthreads();
    const int j0 = max(0, lo - c0), j1 = min(TA_KT, pos - c0 + 1);
#pragma unroll
    for (int i = 0; i < TA_MAX_ACC; i++) {
      const int e = threadIdx.x + i * TA_THREADS;
      if (e < n_out) {
        const int h = e / vdim, c = e - h * vdim;
        const int g = h / rep;
        float a = acc[i] * a_s[h];
        for (int j = j0; j < j1; j++) {
          const T* vr = v_pool + (((long long)page_s[j] * n_kv + g) * page_size + slot_s[j]) * vdim;
          a = fmaf(smix[h * TA_KT + j], to_f32<T>(vr[c]), a);
        }
        acc[i] = a;
      }
    }
    __syncthreads();
  }
  T* orow = out + (long long)t * n_out;
#pragma unroll
  for (int i = 0; i < TA_MAX_ACC; i++) {
    const int e = threadIdx.x + i * TA_THREADS;
    if (e < n_out) orow[e] = from_f32<T>(acc[i] / l_s[e / vdim]);
  }
}

MF_API int mf_attention_talking(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype, int T,
                                int n_heads, int n_kv, int dim, int vdim, const int* positions,
                                const int* seq_of_token, const int* block_table, int bt_stride, int page_size,
                                float scale, float softcap, const float* talk, int window, int chunk,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dim <= 0 || vdim <= 0 || n_kv <= 0 || n_heads % n_kv) return MF_ERR_BAD_ARG;
  if (n_heads * vdim > TA_MAX_ACC * TA_THREADS) return MF_ERR_BAD_ARG;
  const size_t smem = (size_t)(n_heads * dim + 2 * n_heads * TA_KT + n_heads * n_heads + 3 * n_heads) * sizeof(float);
  if (smem > 200 * 1024) return MF_ERR_BAD_ARG;
  mf_count(MF_K_ATTN_TALKING);
#define TA_LAUNCH(TT)                                                                                              \
  do {                                                                                                             \
    if (smem > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(talking_attention_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                             \
      if (e != cudaSuccess) return (int)e;                                                                         \
    }                                                                                                              \
    talking_attention_kernel<TT><<<T, TA_THREADS, smem, stream>>>(                                                 \
        (const TT*)q, (const TT*)k_pool, (const TT*)v_pool, (TT*)out, positions, seq_of_token, block_table,        \
        bt_stride, page_size, n_heads, n_kv, dim, vdim, scale, softcap, talk, window, chunk);                      \
    return (int)cudaGetLastError();                                                                                \
  } while (0)
  if (dtype == MF_F32) TA_LAUNCH(float);
  if (dtype == MF_BF16) TA_LAUNCH(__nv_bfloat16);
#undef TA_LAUNCH
  return MF_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------ biases and the cache write
// qkv [T, nq + nk + nv] (queries, keys, values side by side; 32-bit or the pools' dtype), bias
// [nq + nk + nv] in 32-bit or null.  Queries go to q_out [T, nq]; keys and values of token t
// go to page block_table[seq, p / page_size], slot p % page_size, p = positions[t].
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
biased_kv_store_kernel(const TI* __restrict__ qkv, const float* __restrict__ bias, const int* __restrict__ positions,
                       const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int bt_stride,
                       int page_size, TO* __restrict__ q_out, TO* __restrict__ k_pool, TO* __restrict__ v_pool,
                       int n_heads, int n_kv, int dim, int vdim, int write_kv) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int nq = n_heads * dim, nk = n_kv * dim, nv = n_kv * vdim;
  const TI* row = qkv + (long long)t * (nq + nk + nv);
  for (int i = threadIdx.x; i < nq; i += blockDim.x)
    q_out[(long long)t * nq + i] = from_f32<TO>(to_f32<TI>(row[i]) + (bias ? bias[i] : 0.f));
  if (!write_kv) return;
  const int pos = positions[t], seq = seq_of_token[t];
  const int blk = pos / page_size, slot = pos - blk * page_size;
  const long long page = block_table[(long long)seq * bt_stride + blk];
  for (int i = threadIdx.x; i < nk; i += blockDim.x) {
    const int h = i / dim, d = i - h * dim;
    k_pool[((page * n_kv + h) * page_size + slot) * dim + d] =
        from_f32<TO>(to_f32<TI>(row[nq + i]) + (bias ? bias[nq + i] : 0.f));
  }
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const int h = i / vdim, d = i - h * vdim;
    v_pool[((page * n_kv + h) * page_size + slot) * vdim + d] =
        from_f32<TO>(to_f32<TI>(row[nq + nk + i]) + (bias ? bias[nq + nk + i] : 0.f));
  }
}

MF_API int mf_biased_kv_store(const void* qkv, int in_dtype, const float* bias, const int* positions,
                              const int* seq_of_token, const int* block_table, int bt_stride, int page_size,
                              void* q_out, void* k_pool, void* v_pool, int out_dtype, int T, int n_heads, int n_kv,
                              int dim, int vdim, int write_kv, cudaStream_t stream) {
  if (T <= 0) return 0;
  mf_count(MF_K_KV_STORE);
#define KS_LAUNCH(TI, TO)                                                                                          \
  return (int)launch_dep(biased_kv_store_kernel<TI, TO>, dim3(T), dim3(256), 0, stream, (const TI*)qkv, bias,      \
                         positions, seq_of_token, block_table, bt_stride, page_size, (TO*)q_out, (TO*)k_pool,      \
                         (TO*)v_pool, n_heads, n_kv, dim, vdim, write_kv)
  if (in_dtype == MF_F32 && out_dtype == MF_F32) KS_LAUNCH(float, float);
  if (in_dtype == MF_F32 && out_dtype == MF_BF16) KS_LAUNCH(float, __nv_bfloat16);
  if (in_dtype == MF_BF16 && out_dtype == MF_BF16) KS_LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef KS_LAUNCH
  return MF_ERR_BAD_DTYPE;
}
