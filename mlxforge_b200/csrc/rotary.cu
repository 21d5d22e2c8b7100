// Rotary position encoding in either pairing, fused with the write of keys and values into
// their pages, for mixers whose values are their keys as projected (before the rotation).
//
// One block per token.  A row of `qk` (rows `ld` elements apart) holds the query heads, then the key heads, then (unless the
// values are the keys) the value heads, each head_dim wide.  The first `rot` channels of every
// query and key head are rotated, pair j by the angle position * inv[j]: the pair (u, v) becomes
// (u cos a - v sin a, v cos a + u sin a); the other channels pass.  Rotated queries go to q_out
// [T, n_heads * head_dim], rotated keys to the key pages, and the value pages get the keys before
// the rotation (v_from_k) or the row's value heads.
#include "rotary.cuh"

template <typename T>
__global__ void rope_store_kernel(const T* __restrict__ qk, int ld, int n_heads, int n_kv, int hd, int rot, int layout,
                                  const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                  PagedView pv, const float* __restrict__ inv_f, const double* __restrict__ inv_d,
                                  T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                  int write_kv, int v_from_k) {
  extern __shared__ float cs[];            // [half] cos, [half] sin
  pdl_launch();
  const int t = blockIdx.x;
  const int pos = positions[t], seq = seq_of_token[t];
  const int half = rot >> 1;
  for (int j = threadIdx.x; j < half; j += blockDim.x) rotary_cs(pos, j, inv_f, inv_d, cs[j], cs[half + j]);
  __syncthreads();
  pdl_wait();
  const T* row = qk + (long long)t * ld;
  const int per_head = hd - half;          // `half` pairs and hd - rot channels that pass
  const int heads = n_heads + (write_kv ? n_kv : 0);
  for (int idx = threadIdx.x; idx < heads * per_head; idx += blockDim.x) {
    const int h = idx / per_head, j = idx - h * per_head;
    const T* src = row + (long long)h * hd;
    const bool is_k = h >= n_heads;
    const long long off = is_k ? paged_offset(pv, seq, pos, h - n_heads) : 0;
    T* dst = is_k ? k_pool + off : q_out + ((long long)t * n_heads + h) * hd;
    T* vdst = (is_k && v_from_k) ? v_pool + off : nullptr;
    if (j < half) {
      int a, b;
      rotary_pair(layout, rot, j, a, b);
      const float c = cs[j], s = cs[half + j];
      const float u = to_f32<T>(src[a]), v = to_f32<T>(src[b]);
      dst[a] = from_f32<T>(u * c - v * s);
      dst[b] = from_f32<T>(v * c + u * s);
      if (vdst) {
        vdst[a] = src[a];
        vdst[b] = src[b];
      }
    } else {
      const int ch = rot + (j - half);
      dst[ch] = src[ch];
      if (vdst) vdst[ch] = src[ch];
    }
  }
  if (write_kv && !v_from_k) {
    for (int idx = threadIdx.x; idx < n_kv * hd; idx += blockDim.x) {
      const int h = idx / hd, ch = idx - h * hd;
      v_pool[paged_offset(pv, seq, pos, h) + ch] = row[(long long)(n_heads + n_kv + h) * hd + ch];
    }
  }
}

// bfloat16 with adjacent pairs (2i, 2i + 1), an even head size: a pair is one 32-bit word, and so
// are two channels that pass; every thread moves whole words.
__global__ void __launch_bounds__(256)
rope_store_pairs_bf16_kernel(const __nv_bfloat16* __restrict__ qk, int ld, int n_heads, int n_kv, int hd, int rot,
                             const int* __restrict__ positions, const int* __restrict__ seq_of_token, PagedView pv,
                             const float* __restrict__ inv_f, __nv_bfloat16* __restrict__ q_out,
                             __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool, int write_kv) {
  extern __shared__ float cs[];            // [half] cos, [half] sin
  pdl_launch();
  const int t = blockIdx.x;
  const int pos = positions[t], seq = seq_of_token[t];
  const int half = rot >> 1, words = hd >> 1;
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf((float)pos * inv_f[j], &cs[half + j], &cs[j]);
  __syncthreads();
  pdl_wait();
  const __nv_bfloat16* row = qk + (long long)t * ld;
  const int heads = n_heads + (write_kv ? n_kv : 0);
  for (int idx = threadIdx.x; idx < heads * words; idx += blockDim.x) {
    const int h = idx / words, j = idx - h * words;
    const __nv_bfloat162 in = *reinterpret_cast<const __nv_bfloat162*>(row + (long long)h * hd + 2 * j);
    __nv_bfloat162 o = in;
    if (j < half) {
      const float2 f = __bfloat1622float2(in);
      const float c = cs[j], s = cs[half + j];
      o = __floats2bfloat162_rn(f.x * c - f.y * s, f.y * c + f.x * s);
    }
    if (h < n_heads) {
      *reinterpret_cast<__nv_bfloat162*>(q_out + ((long long)t * n_heads + h) * hd + 2 * j) = o;
    } else {
      const long long off = paged_offset(pv, seq, pos, h - n_heads) + 2 * j;
      *reinterpret_cast<__nv_bfloat162*>(k_pool + off) = o;
      *reinterpret_cast<__nv_bfloat162*>(v_pool + off) = in;          // the values are the keys as projected
    }
  }
}

MF_API int mf_rope_store(const void* qk, int ld, int dtype, int T, int n_heads, int n_kv, int hd, int rot, int layout,
                         const int* positions, const int* seq_of_token, const int* block_table, int bt_stride,
                         int page_size, const float* inv_f, const double* inv_d, void* q_out, void* k_pool,
                         void* v_pool, int write_kv, int v_from_k, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > hd || (rot & 1) || (layout != MF_ROT_HALF && layout != MF_ROT_PAIRS)) return MF_ERR_BAD_ARG;
  if (rot > 0 && !inv_f && !inv_d) return MF_ERR_BAD_ARG;
  PagedView pv{block_table, bt_stride, page_size, n_kv, hd};
  const size_t smem = (size_t)(rot > 0 ? rot : 1) * sizeof(float);
  mf_count(MF_K_ROPE_STORE);
  if (dtype == MF_BF16 && layout == MF_ROT_PAIRS && v_from_k && !inv_d && hd % 2 == 0 && ld % 2 == 0 &&
      (((uintptr_t)qk | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool) & 3) == 0)
    return (int)launch_dep(rope_store_pairs_bf16_kernel, dim3(T), dim3(256), smem, stream, (const __nv_bfloat16*)qk, ld,
                           n_heads, n_kv, hd, rot, positions, seq_of_token, pv, inv_f, (__nv_bfloat16*)q_out,
                           (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, write_kv);
  if (dtype == MF_F32)
    return (int)launch_dep(rope_store_kernel<float>, dim3(T), dim3(256), smem, stream, (const float*)qk, ld, n_heads, n_kv,
                           hd, rot, layout, positions, seq_of_token, pv, inv_f, inv_d, (float*)q_out, (float*)k_pool,
                           (float*)v_pool, write_kv, v_from_k);
  if (dtype == MF_BF16)
    return (int)launch_dep(rope_store_kernel<__nv_bfloat16>, dim3(T), dim3(256), smem, stream,
                           (const __nv_bfloat16*)qk, ld, n_heads, n_kv, hd, rot, layout, positions, seq_of_token, pv, inv_f,
                           inv_d, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, write_kv,
                           v_from_k);
  return MF_ERR_BAD_DTYPE;
}
