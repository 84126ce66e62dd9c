// Attention of single-token steps over ONE cached row per token that is both key and value (attention through a
// latent, queries already carried into the latent's space), on the tensor cores (mma.sync.m16n8k16, float32
// accumulation and softmax).
//
// A cache row holds W bfloat16 values; a score is the whole row against a head's query of W values, and the value
// is the row's first R values.  All heads read the same rows, so a block takes 16 heads of a sequence as the rows of
// one MMA tile and walks a chunk of the sequence's keys in tiles of 64 that lie inside one cache page (cp.async,
// two buffers).  Rows of 1,000 bytes and more are too wide for a warp to keep a head's output in registers, so the
// eight warps split a tile twice: for S = Q K^T each warp takes 8 of the tile's 64 keys (the queries wait in shared
// memory), the maxima and sums of the online softmax are exchanged through shared memory, P goes to shared memory
// as bfloat16, and for O += P V each warp takes an eighth of the value columns over all 64 keys.  The result is
// written normalised (one chunk) or as a partial for `zk_attn_merge` (several).
//
// Shared-memory rows are padded to an odd number of 16-byte pieces, so that the eight rows of an ldmatrix lie in
// different banks whatever W is.  Rows of a tile beyond the last visible key are zero-filled on load, so stale
// cache contents never reach the arithmetic.
#include "common.cuh"
#include <math.h>

#define DL_TK 64
#define DL_WARPS 8
#define DL_THREADS (DL_WARPS * 32)
#define DL_HEADS 16
#define DL_PSTRIDE 72        // bfloat16 per row of P: 9 pieces of 16 bytes

namespace {

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // src-size 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(unsigned r[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned r[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma16816(float c[4], const unsigned a[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&t);
}

// bfloat16 per padded shared-memory row of W values
__host__ __device__ inline int padded_row(int W) { return ((W / 8) | 1) * 8; }

// NV: groups of 8 value columns per warp (even); R <= 64 * NV.
template <int NV>
__global__ void __launch_bounds__(DL_THREADS)
    attn_decode_latent_kernel(const bf16* __restrict__ q, const bf16* __restrict__ cache, bf16* __restrict__ out,
                              float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ seq_start,
                              const int* __restrict__ seq_slot, const int* __restrict__ page_table, int pt_stride,
                              int n_seqs, int H, int W, int R, int page_size, float scale, int num_splits, int split_keys,
                              int parts_always) {
  const int RS = padded_row(W);                       // row stride in shared memory, bfloat16
  const int CHW = W / 8;                              // 16-byte pieces of a row
  extern __shared__ __align__(128) unsigned char smem[];
  bf16* Qs = reinterpret_cast<bf16*>(smem);                                   // [16][RS]
  bf16* Ks0 = Qs + DL_HEADS * RS;                                             // [2][64][RS]
  bf16* Ps = Ks0 + 2 * DL_TK * RS;                                            // [16][DL_PSTRIDE]
  float* red_m = reinterpret_cast<float*>(Ps + DL_HEADS * DL_PSTRIDE);        // [warps][16]
  float* red_l = red_m + DL_WARPS * DL_HEADS;                                 // [warps][16]

  zk_wait_prior();   // nothing of the kernels before is read, and nothing written, above this line
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int b = blockIdx.x, h0 = blockIdx.y * DL_HEADS, split = blockIdx.z;
  const int L = seq_start[b] + 1;  // keys 0 .. L-1; the new token's own row is the last
  int c0 = 0, c1 = L;
  if (num_splits > 1) {
    c0 = split * split_keys;
    c1 = min(L, (split + 1) * split_keys);
  }
  const int* pt = page_table + (size_t)seq_slot[b] * pt_stride;
  const int n_tiles = c1 > c0 ? (c1 - c0 + DL_TK - 1) / DL_TK : 0;

  auto load_tile = [&](int t, int buf) {
    const int kb = c0 + t * DL_TK;          // c0 is a multiple of the tile, a tile lies inside one page
    const int page = pt[kb / page_size];
    const bf16* src = cache + ((size_t)(page < 0 ? 0 : page) * page_size + kb % page_size) * W;
    bf16* dst = Ks0 + (size_t)buf * DL_TK * RS;
    for (int i = tid; i < DL_TK * CHW; i += DL_THREADS) {
      const int r = i / CHW, ch = i - r * CHW;
      const bool valid = page >= 0 && kb + r < c1;
      cp_async16(dst + r * RS + ch * 8, src + (size_t)(valid ? r : 0) * W + ch * 8, valid);
    }
    cp_async_commit();
  };

  // the 16 heads' queries (rows of heads beyond H are zero)
  for (int i = tid; i < DL_HEADS * CHW; i += DL_THREADS) {
    const int r = i / CHW, ch = i - r * CHW;
    const bool valid = h0 + r < H;
    cp_async16(Qs + r * RS + ch * 8, q + ((size_t)b * H + (valid ? h0 + r : 0)) * W + ch * 8, valid);
  }
  cp_async_commit();
  if (n_tiles > 0) load_tile(0, 0);

  const float scale2 = scale * 1.4426950408889634f;     // the softmax runs on base 2
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // rows g and g + 8, the same in every warp
  float o[NV][4];
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[j][i] = 0.f;
  const int KS = W / 16;

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < n_tiles) {
      load_tile(t + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* Ks = Ks0 + (size_t)buf * DL_TK * RS;
    const int kb = c0 + t * DL_TK + 8 * warp;           // this warp's 8 keys of the tile

    // S = Q K^T for 16 heads x 8 keys; one ldmatrix of K serves two k steps
    // (even and odd k steps add into sums of their own, so that one MMA need not wait for the one before it)
    float s[4] = {0.f, 0.f, 0.f, 0.f}, s_odd[4] = {0.f, 0.f, 0.f, 0.f};
    for (int ks = 0; ks < KS; ks += 2) {
      unsigned a[4], a2[4], bfr[4];
      const int chb = 2 * ks + (lane >> 3);
      ldmatrix_x4(bfr, Ks + (8 * warp + (lane & 7)) * RS + (chb < CHW ? chb : 0) * 8);
      ldmatrix_x4(a, Qs + (lane & 15) * RS + (2 * ks + (lane >> 4)) * 8);
      if (ks + 1 < KS) ldmatrix_x4(a2, Qs + (lane & 15) * RS + (2 * ks + 2 + (lane >> 4)) * 8);
      mma16816(s, a, bfr[0], bfr[1]);
      if (ks + 1 < KS) mma16816(s_odd, a2, bfr[2], bfr[3]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i] += s_odd[i];
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int kp = kb + 2 * c + (i & 1);
      s[i] = kp < c1 ? s[i] * scale2 : -INFINITY;
      mx[i >> 1] = fmaxf(mx[i >> 1], s[i]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      if (c == 0) red_m[warp * DL_HEADS + g + 8 * h] = mx[h];
    }
    __syncthreads();
    float alpha[2], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float m_new = m_run[h];
#pragma unroll
      for (int w = 0; w < DL_WARPS; ++w) m_new = fmaxf(m_new, red_m[w * DL_HEADS + g + 8 * h]);
      alpha[h] = m_new == -INFINITY ? 1.f : ex2(m_run[h] - m_new);
      m_run[h] = m_new;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float p = s[i] == -INFINITY ? 0.f : ex2(s[i] - m_run[i >> 1]);
      s[i] = p;
      sum[i >> 1] += p;
    }
    *reinterpret_cast<unsigned*>(Ps + g * DL_PSTRIDE + 8 * warp + 2 * c) = pack_bf16(s[0], s[1]);
    *reinterpret_cast<unsigned*>(Ps + (g + 8) * DL_PSTRIDE + 8 * warp + 2 * c) = pack_bf16(s[2], s[3]);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
      sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
      if (c == 0) red_l[warp * DL_HEADS + g + 8 * h] = sum[h];
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float add = 0.f;
#pragma unroll
      for (int w = 0; w < DL_WARPS; ++w) add += red_l[w * DL_HEADS + g + 8 * h];
      l_run[h] = l_run[h] * alpha[h] + add;
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      o[j][0] *= alpha[0];
      o[j][1] *= alpha[0];
      o[j][2] *= alpha[1];
      o[j][3] *= alpha[1];
    }
    // O += P V: 4 key steps of 16; this warp's value columns are groups warp * NV .. warp * NV + NV - 1
#pragma unroll
    for (int kk = 0; kk < DL_TK / 16; ++kk) {
      unsigned pa[4];
      ldmatrix_x4(pa, Ps + (lane & 15) * DL_PSTRIDE + (2 * kk + (lane >> 4)) * 8);
#pragma unroll
      for (int jn = 0; jn < NV; jn += 2) {
        const int grp = warp * NV + jn;
        if (grp * 8 < R) {            // the same for the whole warp; R is a multiple of 16
          unsigned bfr[4];
          const int r = 16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8;
          ldmatrix_x4_trans(bfr, Ks + r * RS + (grp + (lane >> 4)) * 8);
          mma16816(o[jn], pa, bfr[0], bfr[1]);
          mma16816(o[jn + 1], pa, bfr[2], bfr[3]);
        }
      }
    }
    __syncthreads();  // the tile, P and the exchanged numbers are consumed before the next tile overwrites them
  }
  cp_async_wait<0>();

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int head = h0 + g + 8 * h;
    if (head >= H) continue;
    const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
    const size_t prow = ((size_t)split * n_seqs + b) * H + head;
#pragma unroll
    for (int jn = 0; jn < NV; ++jn) {
      const int col = (warp * NV + jn) * 8 + 2 * c;
      if (col >= R) continue;
      if (num_splits == 1 && !parts_always) {
        *reinterpret_cast<unsigned*>(out + ((size_t)b * H + head) * R + col) = pack_bf16(o[jn][2 * h] * inv, o[jn][2 * h + 1] * inv);
      } else {
        *reinterpret_cast<float2*>(part_o + prow * R + col) = make_float2(o[jn][2 * h], o[jn][2 * h + 1]);
      }
    }
    if ((num_splits > 1 || parts_always) && warp == 0 && c == 0)
      *reinterpret_cast<float2*>(part_ml + prow * 2) = make_float2(m_run[h] * 0.6931471805599453f, l_run[h]);
  }
}

size_t smem_bytes(int W) {
  return (size_t)(DL_HEADS + 2 * DL_TK) * padded_row(W) * 2 + DL_HEADS * DL_PSTRIDE * 2 + 2 * DL_WARPS * DL_HEADS * 4;
}

template <int NV>
int launch(const void* q, const void* cache, void* out, float* part_o, float* part_ml, const int* seq_start,
           const int* seq_slot, const int* page_table, int pt_stride, int n_seqs, int H, int W, int R, int page_size,
           float scale, int num_splits, int split_keys, cudaStream_t stream) {
  auto kern = attn_decode_latent_kernel<NV>;
  const size_t smem = smem_bytes(W);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(n_seqs, (H + DL_HEADS - 1) / DL_HEADS, num_splits);
  return zk_launch_dependent(kern, grid, dim3(DL_THREADS), smem, stream, (const bf16*)q, (const bf16*)cache, (bf16*)out,
                             part_o, part_ml, seq_start, seq_slot, page_table, pt_stride, n_seqs, H, W, R, page_size, scale,
                             num_splits, split_keys, (part_o && part_ml) ? 1 : 0);
}

}  // namespace

extern "C" {

// Rows of W values of which the first R are the value: W and R multiples of 16, R <= W, R <= 512, pages of a
// multiple of 64 tokens, and the tiles must fit in shared memory (W up to 768).
int zk_attn_decode_latent_takes(int H, int W, int R, int page_size) {
  if (H <= 0 || W <= 0 || R <= 0 || W % 16 || R % 16 || R > W || R > 512) return 0;
  return page_size % DL_TK == 0 && smem_bytes(W) <= 220 * 1024;
}

// q [n_seqs, H * W] bfloat16 (row b = sequence b); cache [pages, 1, page_size, W]; out [n_seqs, H * R]; partials as
// for zk_attn_fwd when num_splits > 1 (rows ordered (split, sequence, head), R values each).  With partials given and
// num_splits = 1 the unnormalised sums go there all the same and `out` is not written: the caller's merge then
// normalises them, for instance with a sink as one more term of the denominator.
int zk_attn_decode_latent(const void* q, const void* cache, void* out, float* part_o, float* part_ml, const int* seq_start,
                          const int* seq_slot, const int* page_table, int pt_stride, int n_seqs, int H, int W, int R,
                          int page_size, float scale, int num_splits, int split_keys, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (!zk_attn_decode_latent_takes(H, W, R, page_size) || num_splits < 1) return ZK_EINVAL;
  if (num_splits > 1 && (split_keys <= 0 || split_keys % DL_TK || !part_o || !part_ml)) return ZK_EINVAL;
  if (num_splits > 65535 || (H + DL_HEADS - 1) / DL_HEADS > 65535) return ZK_EINVAL;
#define ZK_DL(NVV)                                                                                                     \
  return launch<NVV>(q, cache, out, part_o, part_ml, seq_start, seq_slot, page_table, pt_stride, n_seqs, H, W, R, page_size, \
                     scale, num_splits, split_keys, stream)
  if (R <= 128) ZK_DL(2);
  if (R <= 256) ZK_DL(4);
  ZK_DL(8);
#undef ZK_DL
}

}  // extern "C"
