// Attention with talking heads for portions of prompts, bfloat16, on the tensor cores.
//
// The formulas are those of attention_talking.cu.  The mixing of the heads' scores before the
// softmax couples all heads of a (query, key) pair, so a block owns a tile of 16 queries of one
// sequence with ALL heads, one warp per head, and walks over the keys in tiles of 32 that start
// at multiples of 32 (the order of every sum depends on positions only).  Per key tile:
//
//   1. warp h:  S_h = Q_h K_g(h)^T (mma.sync m16n8k16, 32-bit accumulators), scale, soft cap,
//               stored to shared memory in 32-bit;
//   2. all threads, four keys of one query each: s'_h = sum_g talk[h, g] s_g for every h, in
//               32-bit FMAs, and the mask (causal, chunk, window, length), in place;
//   3. warp h:  online softmax of its mixed scores (32-bit), P_h rounded to bfloat16 as the
//               A operand, O_h += P_h V_g(h).
//
// Keys and values of a tile come in by cp.async (16 bytes a copy) after the two pages of the
// tile's granules have been looked up once, so a tile waits for one round trip to memory and
// not for one per piece.
//
// Decoding (one query per sequence) runs the same kernel with the keys cut into splits of
// TT_SPLIT_TILES tiles that start at multiples of that many tiles: a block per (sequence, split)
// writes its unnormalised output with its running maximum and sum, and a merge kernel joins the
// splits.  A split's range depends on positions only.  Portions of prompts whose queries see more
// than TT_PREFILL_SPLIT_TILES tiles of keys are cut the same way (the last tile of queries of a
// long prompt would otherwise walk all its keys alone while the blocks of the first tiles are
// long done).
//
// Steps 1 and 3 are tensor-core work of 2 * 16 * 32 * (dim + vdim) MACs per head; step 2 is
// H^2 * 512 32-bit FMAs per tile plus a tanh and an exponential per score, which is what bounds
// the kernel: the mixing has to stay 32-bit.
#include "common.cuh"

#define TT_BM 16
#define TT_BN 32
#define TT_SPAD 4          // floats of padding per row of the score tile
#define TT_SPLIT_TILES 4   // key tiles per split when decoding (128 keys)
#define TT_PREFILL_SPLIT_TILES 32   // and for portions of prompts (1024 keys)

__device__ __forceinline__ void tt_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void tt_ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* p) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void tt_cp_async16(void* smem, const void* gmem) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(addr), "l"(gmem) : "memory");
}
__device__ __forceinline__ void tt_cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t tt_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// tanh in 32-bit arithmetic through one exponential: (1 - e^{-2|x|}) / (1 + e^{-2|x|})
__device__ __forceinline__ float tt_tanh(float x) {
  const float t = __expf(-2.0f * fabsf(x));
  return copysignf(__fdividef(1.0f - t, 1.0f + t), x);
}

struct TtArgs {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k_pool;
  const __nv_bfloat16* v_pool;
  __nv_bfloat16* out;
  const int* seq_q_start;
  const int* seq_q_len;
  const int* seq_ctx_len;
  const int* block_table;
  const float* talk;
  int table_row0, bt_stride, page_size, n_heads, n_kv, dim;
  float scale, softcap;
  int window, chunk;
  int splits;               // 0: every block walks all its keys; else gridDim.z splits of split_tiles tiles
  int split_tiles;
  float* part_o;            // [rows, splits, H, VDIM] unnormalised outputs of the splits
  float* part_ml;           // [rows, splits, H, 2]    running maximum and sum
};

template <int VDIM, int MAXH>
__global__ void __launch_bounds__(32 * MAXH)
talking_attention_tc_kernel(const TtArgs a) {
  extern __shared__ __align__(16) unsigned char tt_smem[];
  const int H = a.n_heads, G = a.n_kv, dim = a.dim;
  const int rep = H / G;
  const int seq = blockIdx.y;
  const int q_len = a.seq_q_len[seq];
  const int row0 = blockIdx.x * TT_BM;
  if (row0 >= q_len) return;
  const int q_start = a.seq_q_start[seq], ctx = a.seq_ctx_len[seq];
  const int pos0 = ctx - q_len + row0;                       // position of the tile's first query
  const int rows = min(TT_BM, q_len - row0);
  const int* table = a.block_table + (long long)(a.table_row0 + seq) * a.bt_stride;

  const int qs_ld = dim + 8, vs_ld = VDIM + 8, sc_ld = TT_BN + TT_SPAD;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(tt_smem);            // [H][16][qs_ld]
  __nv_bfloat16* Ks = Qs + (size_t)H * TT_BM * qs_ld;                       // [G][32][qs_ld]
  __nv_bfloat16* Vs = Ks + (size_t)G * TT_BN * qs_ld;                       // [G][32][vs_ld]
  float* sc = reinterpret_cast<float*>(Vs + (size_t)G * TT_BN * vs_ld);     // [H][16][sc_ld]
  float* tk = sc + (size_t)H * TT_BM * sc_ld;                               // [H from][MAXH to], zero beyond H

  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5;          // warp = head
  const int r0 = lane >> 2, c2 = (lane & 3) * 2;

  // queries of the tile, all heads: rows beyond the portion are zero
  const int dv8 = dim / 8;
  for (int i = tid; i < H * TT_BM * dv8; i += nthreads) {
    const int h = i / (TT_BM * dv8), rem = i - h * TT_BM * dv8;
    const int r = rem / dv8, c = (rem - r * dv8) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows) v = *reinterpret_cast<const uint4*>(a.q + ((long long)(q_start + row0 + r) * H + h) * dim + c);
    *reinterpret_cast<uint4*>(Qs + ((size_t)h * TT_BM + r) * qs_ld + c) = v;
  }
  for (int i = tid; i < H * MAXH; i += nthreads) {
    const int g = i / MAXH, h = i - g * MAXH;
    tk[i] = h < H ? (a.talk ? a.talk[h * H + g] : (h == g ? 1.f : 0.f)) : 0.f;
  }

  // the first key any query of the tile sees: that of its first query
  int lo0 = 0;
  if (a.window > 0) lo0 = max(lo0, pos0 - a.window + 1);
  if (a.chunk > 0) lo0 = max(lo0, pos0 / a.chunk * a.chunk);
  const int pos_last = pos0 + rows - 1;

  float o[VDIM / 8][4];
#pragma unroll
  for (int i = 0; i < VDIM / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int g_own = warp / rep;
  const bool has_head = warp < H;

  // how this thread walks over the pieces of a key tile
  int kc, kcs, kr0, krs;
  if (nthreads % dv8 == 0) {
    kc = (tid % dv8) * 8; kcs = dim; kr0 = tid / dv8; krs = nthreads / dv8;
  } else {                   // a row at a time, its pieces in turn
    kc = 0; kcs = 8; kr0 = tid; krs = nthreads;
  }
  int k_first = (lo0 / TT_BN) * TT_BN, k_last = pos_last;
  if (a.splits > 0) {      // this block's share: tiles [z, z + 1) * TT_SPLIT_TILES of the sequence
    const int span = a.split_tiles * TT_BN;
    const int first_split = k_first / span;
    k_first = max(k_first, (first_split + (int)blockIdx.z) * span);
    k_last = min(k_last, (first_split + (int)blockIdx.z + 1) * span - 1);
  }
  for (int k0 = k_first; k0 <= k_last; k0 += TT_BN) {
    __syncthreads();       // the tile before is done with Ks, Vs and sc (and Qs, tk are written)
    // keys and values of the tile: two granules of 16 positions, each inside one page
    long long pg[TT_BN / 16];
    int sl[TT_BN / 16];
#pragma unroll
    for (int gq = 0; gq < TT_BN / 16; gq++) {
      const int p0 = k0 + 16 * gq;
      const int blk = p0 / a.page_size;
      sl[gq] = p0 - blk * a.page_size;
      pg[gq] = (p0 <= pos_last && p0 + 15 >= lo0) ? (long long)table[blk] : -1;
    }
    // a thread copies the same 16-byte column of every row it takes (kc, row stride krs), where the
    // block's threads divide evenly among a row's pieces; else piece by piece
    for (int row = kr0; row < G * TT_BN; row += krs) {
      for (int c = kc; c < dim; c += kcs) {
        const int g = row / TT_BN, j = row - g * TT_BN;
        const int pj = k0 + j;
        __nv_bfloat16* dst = Ks + (size_t)row * qs_ld + c;
        const long long page = (j >> 4) ? pg[1] : pg[0];
        const int slot = ((j >> 4) ? sl[1] : sl[0]) + (j & 15);
        if (pj >= lo0 && pj <= pos_last && page >= 0)
          tt_cp_async16(dst, a.k_pool + ((page * G + g) * a.page_size + slot) * dim + c);
        else
          *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
    for (int i = tid; i < G * TT_BN * (VDIM / 8); i += nthreads) {
      const int row = i / (VDIM / 8), c = (i - row * (VDIM / 8)) * 8;
      const int g = row / TT_BN, j = row - g * TT_BN;
      const int pj = k0 + j;
      __nv_bfloat16* dst = Vs + (size_t)row * vs_ld + c;
      const long long page = (j >> 4) ? pg[1] : pg[0];
      const int slot = ((j >> 4) ? sl[1] : sl[0]) + (j & 15);
      if (pj >= lo0 && pj <= pos_last && page >= 0)
        tt_cp_async16(dst, a.v_pool + ((page * G + g) * a.page_size + slot) * VDIM + c);
      else
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    tt_cp_async_wait_all();
    __syncthreads();

    // 1. raw scores of this warp's head
    if (has_head) {
      float s[TT_BN / 8][4];
#pragma unroll
      for (int nt = 0; nt < TT_BN / 8; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
      const __nv_bfloat16* qh = Qs + (size_t)warp * TT_BM * qs_ld;
      const __nv_bfloat16* kg = Ks + (size_t)g_own * TT_BN * qs_ld;
      for (int kk = 0; kk < dim; kk += 16) {
        uint32_t af[4];
        af[0] = *reinterpret_cast<const uint32_t*>(qh + (size_t)r0 * qs_ld + kk + c2);
        af[1] = *reinterpret_cast<const uint32_t*>(qh + (size_t)(r0 + 8) * qs_ld + kk + c2);
        af[2] = *reinterpret_cast<const uint32_t*>(qh + (size_t)r0 * qs_ld + kk + 8 + c2);
        af[3] = *reinterpret_cast<const uint32_t*>(qh + (size_t)(r0 + 8) * qs_ld + kk + 8 + c2);
#pragma unroll
        for (int nt = 0; nt < TT_BN / 8; nt++) {
          const __nv_bfloat16* kr = kg + (size_t)(nt * 8 + r0) * qs_ld + kk + c2;
          tt_mma(s[nt], af, *reinterpret_cast<const uint32_t*>(kr), *reinterpret_cast<const uint32_t*>(kr + 8));
        }
      }
      float* sh = sc + (size_t)warp * TT_BM * sc_ld;
#pragma unroll
      for (int nt = 0; nt < TT_BN / 8; nt++) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
          float v = s[nt][e] * a.scale;
          if (a.softcap > 0.f) v = a.softcap * tt_tanh(v / a.softcap);
          s[nt][e] = v;
        }
        *reinterpret_cast<float2*>(sh + (size_t)r0 * sc_ld + nt * 8 + c2) = make_float2(s[nt][0], s[nt][1]);
        *reinterpret_cast<float2*>(sh + (size_t)(r0 + 8) * sc_ld + nt * 8 + c2) = make_float2(s[nt][2], s[nt][3]);
      }
    }
    __syncthreads();

    // 2. the heads mixed and the mask, two keys of one query per thread and pass
    for (int pair = tid; pair < rows * (TT_BN / 2); pair += nthreads) {
      const int r = pair / (TT_BN / 2), j2 = (pair - r * (TT_BN / 2)) * 2;
      float acc[MAXH][2];
#pragma unroll
      for (int h = 0; h < MAXH; h++) acc[h][0] = acc[h][1] = 0.f;
      if (a.talk) {
        for (int g = 0; g < H; g++) {
          const float2 sg = *reinterpret_cast<const float2*>(sc + ((size_t)g * TT_BM + r) * sc_ld + j2);
          const float4* tg = reinterpret_cast<const float4*>(tk + g * MAXH);
#pragma unroll
          for (int h4 = 0; h4 < MAXH / 4; h4++) {       // heads beyond H have weight zero and are not stored
            const float4 t = tg[h4];
            acc[4 * h4][0] = fmaf(t.x, sg.x, acc[4 * h4][0]);
            acc[4 * h4][1] = fmaf(t.x, sg.y, acc[4 * h4][1]);
            acc[4 * h4 + 1][0] = fmaf(t.y, sg.x, acc[4 * h4 + 1][0]);
            acc[4 * h4 + 1][1] = fmaf(t.y, sg.y, acc[4 * h4 + 1][1]);
            acc[4 * h4 + 2][0] = fmaf(t.z, sg.x, acc[4 * h4 + 2][0]);
            acc[4 * h4 + 2][1] = fmaf(t.z, sg.y, acc[4 * h4 + 2][1]);
            acc[4 * h4 + 3][0] = fmaf(t.w, sg.x, acc[4 * h4 + 3][0]);
            acc[4 * h4 + 3][1] = fmaf(t.w, sg.y, acc[4 * h4 + 3][1]);
          }
        }
      } else {
#pragma unroll
        for (int h = 0; h < MAXH; h++) {
          if (h < H) {
            const float2 sg = *reinterpret_cast<const float2*>(sc + ((size_t)h * TT_BM + r) * sc_ld + j2);
            acc[h][0] = sg.x; acc[h][1] = sg.y;
          }
        }
      }
      const int pi = pos0 + r;
      int lo = 0;
      if (a.window > 0) lo = max(lo, pi - a.window + 1);
      if (a.chunk > 0) lo = max(lo, pi / a.chunk * a.chunk);
      const int pj = k0 + j2;
      const bool ok0 = pj >= lo && pj <= pi, ok1 = pj + 1 >= lo && pj + 1 <= pi;
#pragma unroll
      for (int h = 0; h < MAXH; h++) {
        if (h < H)
          *reinterpret_cast<float2*>(sc + ((size_t)h * TT_BM + r) * sc_ld + j2) =
              make_float2(ok0 ? acc[h][0] : -INFINITY, ok1 ? acc[h][1] : -INFINITY);
      }
    }
    __syncthreads();

    // 3. softmax of the mixed scores and the product with the values
    if (has_head) {
      const float* sh = sc + (size_t)warp * TT_BM * sc_ld;
      float s[TT_BN / 8][4];
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < TT_BN / 8; nt++) {
        float2 x = *reinterpret_cast<const float2*>(sh + (size_t)r0 * sc_ld + nt * 8 + c2);
        float2 y = *reinterpret_cast<const float2*>(sh + (size_t)(r0 + 8) * sc_ld + nt * 8 + c2);
        if (r0 >= rows) x = make_float2(-INFINITY, -INFINITY);          // rows beyond the portion were not mixed
        if (r0 + 8 >= rows) y = make_float2(-INFINITY, -INFINITY);
        s[nt][0] = x.x; s[nt][1] = x.y; s[nt][2] = y.x; s[nt][3] = y.y;
        mx[0] = fmaxf(mx[0], fmaxf(x.x, x.y));
        mx[1] = fmaxf(mx[1], fmaxf(y.x, y.y));
      }
      float alpha[2];
#pragma unroll
      for (int e = 0; e < 2; e++) {
        mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 1));
        mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 2));
        const float m_new = fmaxf(m_run[e], mx[e]);
        alpha[e] = (m_run[e] == -INFINITY) ? 0.f : __expf(m_run[e] - m_new);
        m_run[e] = m_new;
      }
      float sum[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < TT_BN / 8; nt++) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const float m = m_run[e >> 1];
          const float p = (s[nt][e] == -INFINITY) ? 0.f : __expf(s[nt][e] - m);
          s[nt][e] = p;
          sum[e >> 1] += p;
        }
      }
      l_run[0] = l_run[0] * alpha[0] + sum[0];
      l_run[1] = l_run[1] * alpha[1] + sum[1];
#pragma unroll
      for (int i = 0; i < VDIM / 8; i++) {
        o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
        o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
      }
      const __nv_bfloat16* vg = Vs + (size_t)g_own * TT_BN * vs_ld;
#pragma unroll
      for (int ks = 0; ks < TT_BN / 16; ks++) {
        uint32_t pf[4];
        pf[0] = tt_pack(s[2 * ks][0], s[2 * ks][1]);
        pf[1] = tt_pack(s[2 * ks][2], s[2 * ks][3]);
        pf[2] = tt_pack(s[2 * ks + 1][0], s[2 * ks + 1][1]);
        pf[3] = tt_pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
        for (int nt = 0; nt < VDIM / 8; nt++) {
          uint32_t b0, b1;
          tt_ldmatrix_x2_trans(b0, b1, vg + (size_t)(ks * 16 + (lane & 15)) * vs_ld + nt * 8);
          tt_mma(o[nt], pf, b0, b1);
        }
      }
    }
  }

  if (has_head) {
#pragma unroll
    for (int e = 0; e < 2; e++) {
      l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 1);
      l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 2);
    }
    if (a.splits > 0) {      // the split's unnormalised rows with their maximum and sum
#pragma unroll
      for (int half = 0; half < 2; half++) {
        const int r = r0 + 8 * half;
        if (r < rows) {
          const long long slot = ((long long)(q_start + row0 + r) * a.splits + blockIdx.z) * H + warp;
#pragma unroll
          for (int nt = 0; nt < VDIM / 8; nt++)
            *reinterpret_cast<float2*>(a.part_o + slot * VDIM + nt * 8 + c2) =
                make_float2(o[nt][2 * half], o[nt][2 * half + 1]);
          if (c2 == 0) {
            a.part_ml[slot * 2] = m_run[half];
            a.part_ml[slot * 2 + 1] = l_run[half];
          }
        }
      }
      return;
    }
    const float inv0 = 1.0f / l_run[0], inv1 = 1.0f / l_run[1];
#pragma unroll
    for (int nt = 0; nt < VDIM / 8; nt++) {
      if (r0 < rows)
        *reinterpret_cast<__nv_bfloat162*>(a.out + ((long long)(q_start + row0 + r0) * H + warp) * VDIM + nt * 8 + c2) =
            __floats2bfloat162_rn(o[nt][0] * inv0, o[nt][1] * inv0);
      if (r0 + 8 < rows)
        *reinterpret_cast<__nv_bfloat162*>(a.out + ((long long)(q_start + row0 + r0 + 8) * H + warp) * VDIM + nt * 8 + c2) =
            __floats2bfloat162_rn(o[nt][2] * inv1, o[nt][3] * inv1);
    }
  }
}

static size_t tt_smem_bytes(int H, int G, int dim, int vdim) {
  return (size_t)(H * TT_BM + G * TT_BN) * (dim + 8) * 2 + (size_t)G * TT_BN * (vdim + 8) * 2 +
         (size_t)H * TT_BM * (TT_BN + TT_SPAD) * 4 + (size_t)H * 16 * 4;
}

// 1 if the kernel takes these sizes
MF_API int mf_attention_talking_tc_ok(int n_heads, int n_kv, int dim, int vdim, int page_size) {
  if (n_heads < 1 || n_heads > 16 || n_kv < 1 || n_heads % n_kv) return 0;
  if (dim % 16 || dim < 16 || dim > 256) return 0;
  if (vdim != 32 && vdim != 64 && vdim != 96 && vdim != 128) return 0;
  if (page_size % 16) return 0;
  return tt_smem_bytes(n_heads, n_kv, dim, vdim) <= 200 * 1024 ? 1 : 0;
}

// out[t, h] = sum_z o_z e^{m_z - m} / sum_z l_z e^{m_z - m}, the splits in their order
__global__ void __launch_bounds__(128)
talking_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                               __nv_bfloat16* __restrict__ out, int splits, int H, int vdim, int first_row) {
  const int t = first_row + blockIdx.x, h = blockIdx.y;
  const float* ml = part_ml + ((long long)t * splits * H + h) * 2;
  float m = -INFINITY;
  for (int z = 0; z < splits; z++) m = fmaxf(m, ml[(long long)z * H * 2]);
  float l = 0.f;
  for (int z = 0; z < splits; z++) {
    const float mz = ml[(long long)z * H * 2];
    if (mz != -INFINITY) l += ml[(long long)z * H * 2 + 1] * __expf(mz - m);
  }
  const float inv = 1.0f / l;
  for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
    float acc = 0.f;
    for (int z = 0; z < splits; z++) {
      const float mz = ml[(long long)z * H * 2];
      if (mz != -INFINITY) acc += part_o[(((long long)t * splits + z) * H + h) * vdim + c] * __expf(mz - m);
    }
    out[((long long)t * H + h) * vdim + c] = __float2bfloat16_rn(acc * inv);
  }
}

template <int VDIM, int MAXH>
static int tt_launch(const TtArgs& a, int n_seqs, int max_q_len, cudaStream_t stream) {
  const size_t smem = tt_smem_bytes(a.n_heads, a.n_kv, a.dim, VDIM);
  static DeviceOnce once;
  const int d = mf_current_device();
  if (d < 0) return MF_ERR_BAD_ARG;
  if (!once.done[d]) {
    cudaError_t e = cudaFuncSetAttribute(talking_attention_tc_kernel<VDIM, MAXH>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    once.done[d] = true;
  }
  dim3 grid((max_q_len + TT_BM - 1) / TT_BM, n_seqs, a.splits > 0 ? a.splits : 1);
  const int warps = a.n_heads < 4 ? 4 : a.n_heads;       // at least four warps for the loads and the mixing
  talking_attention_tc_kernel<VDIM, MAXH><<<grid, 32 * warps, smem, stream>>>(a);
  return (int)cudaGetLastError();
}

// The sequences described by the three per-sequence arrays start at row `table_row0` of the
// block table; q and out are the whole step's [T, n_heads * dim] and [T, n_heads * vdim].
MF_API int mf_attention_talking_tc(const void* q, const void* k_pool, const void* v_pool, void* out,
                                   const int* seq_q_start, const int* seq_q_len, const int* seq_ctx_len,
                                   int table_row0, int n_seqs, int max_q_len, int n_heads, int n_kv, int dim, int vdim,
                                   const int* block_table, int bt_stride, int page_size, float scale, float softcap,
                                   const float* talk, int window, int chunk, int splits, float* part_o, float* part_ml,
                                   int first_row, int n_rows, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return 0;
  if (!mf_attention_talking_tc_ok(n_heads, n_kv, dim, vdim, page_size) || n_seqs > 65535 || splits < 0 || splits > 65535)
    return MF_ERR_BAD_ARG;
  TtArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out,
           seq_q_start, seq_q_len, seq_ctx_len, block_table, talk, table_row0, bt_stride, page_size, n_heads, n_kv, dim,
           scale, softcap, window, chunk, splits, TT_PREFILL_SPLIT_TILES, part_o, part_ml};
  mf_count(MF_K_ATTN_TALKING_TC);
  int rc = MF_ERR_BAD_ARG;
#define TT_CASE(VD)                                                         \
  if (vdim == VD)                                                           \
    rc = n_heads <= 8 ? tt_launch<VD, 8>(a, n_seqs, max_q_len, stream) : tt_launch<VD, 16>(a, n_seqs, max_q_len, stream);
  TT_CASE(32)
  TT_CASE(64)
  TT_CASE(96)
  TT_CASE(128)
#undef TT_CASE
  if (rc != 0 || splits == 0) return rc;
  // the rows of the portions are rows first_row .. first_row + n_rows of the step
  mf_count(MF_K_ATTN_TALKING_MERGE);
  talking_attention_merge_kernel<<<dim3(n_rows, n_heads), 128, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, splits,
                                                                        n_heads, vdim, first_row);
  return (int)cudaGetLastError();
}

// Splits of a launch for portions of prompts whose queries see at most `max_keys` keys (0: none needed).
MF_API int mf_attention_talking_prefill_splits(int max_keys) {
  const int tiles = (max_keys + TT_BN - 1) / TT_BN + 1;
  if (tiles <= TT_PREFILL_SPLIT_TILES + 1) return 0;
  return (tiles + TT_PREFILL_SPLIT_TILES - 1) / TT_PREFILL_SPLIT_TILES + 1;
}

// Splits that a decode launch needs when no query sees more than `max_keys` keys.
MF_API int mf_attention_talking_splits(int max_keys) {
  const int tiles = (max_keys + TT_BN - 1) / TT_BN + 1;       // a range of keys may straddle one tile more
  return (tiles + TT_SPLIT_TILES - 1) / TT_SPLIT_TILES + 1;   // and one split more
}

// One query per sequence (the newest token of each), keys cut into splits; q and out hold the
// n_seqs tokens, row t the token of row t of the block table.  part_o needs
// n_seqs * splits * n_heads * vdim floats, part_ml n_seqs * splits * n_heads * 2.
MF_API int mf_attention_talking_decode(const void* q, const void* k_pool, const void* v_pool, void* out,
                                       const int* seq_q_start, const int* seq_q_len, const int* seq_ctx_len, int n_seqs,
                                       int n_heads, int n_kv, int dim, int vdim, const int* block_table, int bt_stride,
                                       int page_size, float scale, float softcap, const float* talk, int window,
                                       int chunk, int splits, float* part_o, float* part_ml, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (!mf_attention_talking_tc_ok(n_heads, n_kv, dim, vdim, page_size) || n_seqs > 65535 || splits < 1 || splits > 65535)
    return MF_ERR_BAD_ARG;
  TtArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out,
           seq_q_start, seq_q_len, seq_ctx_len, block_table, talk, 0, bt_stride, page_size, n_heads, n_kv, dim,
           scale, softcap, window, chunk, splits, TT_SPLIT_TILES, part_o, part_ml};
  mf_count(MF_K_ATTN_TALKING_TC);
  int rc = MF_ERR_BAD_ARG;
#define TT_CASE(VD)                                                         \
  if (vdim == VD) rc = n_heads <= 8 ? tt_launch<VD, 8>(a, n_seqs, 1, stream) : tt_launch<VD, 16>(a, n_seqs, 1, stream);
  TT_CASE(32)
  TT_CASE(64)
  TT_CASE(96)
  TT_CASE(128)
#undef TT_CASE
  if (rc != 0) return rc;
  mf_count(MF_K_ATTN_TALKING_MERGE);
  talking_attention_merge_kernel<<<dim3(n_seqs, n_heads), 128, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, splits,
                                                                         n_heads, vdim, 0);
  return (int)cudaGetLastError();
}
