// Attention whose keys and values are expanded from one latent vector per token.
//
// Per token the cache holds ONE row [c (r) | k_rot (p)]: c the RMS-normalised latent, k_rot a rotated key part
// that all heads share.  With W_uk [H*d, r] and W_uv [H*e, r] the expansions k_h = W_uk,h c and v_h = W_uv,h c are
// never made for cached tokens: a head's query is carried into the latent's space, q'_h = [W_uk,h^T q_h | rot(q_rot,h)],
// so that q'_h . row = q_h . k_h + rot(q_rot,h) . k_rot, the softmax weights are applied to c itself, and W_uv,h
// expands the weighted sum afterwards.  Attention is then multi-query attention over rows of r + p values whose
// first r values are also the "value".
//
// (1) latent_prepare_kernel: norm of the latent, rotation of the shared key part, cache write; rotation of the
//     queries' rotated parts into their place behind the r latent-space columns.
//     A prompt step that starts its sequences (nothing cached before it) is cheaper the other way round: every
//     head's keys and values ARE expanded for the step's own tokens (one contraction of c against [W_uk; W_uv]),
//     and (1b) latent_pack_kernel lays queries, keys and values out, padded to the widths the tensor-core prompt
//     kernel takes, in rows ordered like a cache's pages for this step alone.  The scores then cost d + p
//     multiplications a key, not r + p.  A prompt step that continues its sequences does the same over ALL their
//     tokens: latent_gather_kernel packs the cached latents, the contraction expands them once more, and the shared
//     key part is read back from the cache rows.
// (2) head_gemm_kernel: out[t, h, :] = a[t, h, :] W[h]^T for few tokens, weights streamed once (the two per-head
//     steps around attention in single-token steps), with an optional sigmoid gate per (token, head).
#include "common.cuh"
#include <math.h>

#define LAT_THREADS 256

// Block (t, 0): rotated query parts.  q [n, H * (d + p)] as the projection left it (head by head [d | p]); the
// rotated p entries of head h go to q_full[t, h, r .. r + p) (rows of H * (r + p); the first r columns of every
// head are written by the contraction that follows).  Block (t, 1): the token's cache row from dkv (float32, rows
// `ld_dkv` apart): [rms(dkv[:r]) * w | rot(dkv[r : r + p])].  Pairs (i, i + p/2), angle = float(pos) * inv_freq[i].
// q_full null: block (t, 0) has nothing to do.  c_out [n, r] (or null): the normalised latent once more, packed.
template <typename T>
__global__ void __launch_bounds__(LAT_THREADS)
    latent_prepare_kernel(const T* __restrict__ q, T* __restrict__ q_full, const float* __restrict__ dkv, int ld_dkv,
                          const float* __restrict__ c_w, const float* __restrict__ inv_freq, T* __restrict__ cache,
                          const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                          const int* __restrict__ seq_slot, const int* __restrict__ page_table, int pt_stride, int H,
                          int d, int p, int r, float eps, int page_size, int write_kv, int* status,
                          T* __restrict__ c_out) {
  __shared__ float scratch[32];
  zk_let_next_start();
  zk_wait_prior();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int pos = tok_pos[t];
  const int half = p >> 1;
  if (blockIdx.y == 0) {
    if (!q_full) return;
    for (int idx = tid; idx < H * half; idx += LAT_THREADS) {
      const int h = idx / half, i = idx - h * half;
      const T* src = q + ((size_t)t * H + h) * (d + p) + d;
      const float ang = (float)pos * inv_freq[i];
      const float c = cosf(ang), sn = sinf(ang);
      const float u = to_f32(src[i]), v = to_f32(src[i + half]);
      T* dst = q_full + ((size_t)t * H + h) * (r + p) + r;
      dst[i] = from_f32<T>(u * c - v * sn);
      dst[i + half] = from_f32<T>(u * sn + v * c);
    }
    return;
  }
  if (!write_kv && !c_out) return;
  const float* src = dkv + (size_t)t * ld_dkv;
  float ss = 0.f;
  for (int i = tid; i < r; i += LAT_THREADS) ss = fmaf(src[i], src[i], ss);
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)r + eps);
  if (c_out)
    for (int i = tid; i < r; i += LAT_THREADS) c_out[(size_t)t * r + i] = from_f32<T>((src[i] * scale) * c_w[i]);
  if (!write_kv) return;
  const int page = page_table[(size_t)seq_slot[tok_seq[t]] * pt_stride + pos / page_size];
  if (page < 0) {
    if (tid == 0) atomicExch(status, 2);
    return;
  }
  T* row = cache + ((size_t)page * page_size + pos % page_size) * (r + p);
  for (int i = tid; i < r; i += LAT_THREADS) row[i] = from_f32<T>((src[i] * scale) * c_w[i]);
  for (int i = tid; i < half; i += LAT_THREADS) {
    const float ang = (float)pos * inv_freq[i];
    const float c = cosf(ang), sn = sinf(ang);
    const float u = src[r + i], v = src[r + i + half];
    row[r + i] = from_f32<T>(u * c - v * sn);
    row[r + i + half] = from_f32<T>(u * sn + v * c);
  }
}

// Queries, keys and values of a prompt step laid out for attention over rows of the step's own (no cache).
// Block (t, 0), t < n_q: a step token.  q [n_q, H * (d + p)] as projected -> q_pad [n_q, H * HD] =
// [q_h[:d] | rot(q_h[d:]) | 0], rotated by tok_pos[t].
// Block (j, 1), j < n_kv: a key/value token (kv_seq[j], kv_pos[j]): the step's tokens themselves when its sequences
// start at position 0, else every position of the step's sequences up to their last token.  kvx rows `ld_kvx` apart:
// [H * d expanded unrotated keys | H * e expanded values] of token j.  The shared rotated key part comes from
// dkv[j] (float32, rows `ld_dkv` apart, entries r.., rotated here) or, with `cache` given, from the token's cache row
// (entries r.., already rotated).  Written at row (page, h, pos % page_size), page = seq_page0[sequence] + pos /
// page_size: k_rows [pages, H, page_size, HD] = [k_h | rot(k_rot) | 0], v_rows [pages, H, page_size, HDV] = [v_h | 0].
template <typename T>
__global__ void __launch_bounds__(LAT_THREADS)
    latent_pack_kernel(const T* __restrict__ q, const T* __restrict__ kvx, int ld_kvx, const float* __restrict__ dkv,
                       int ld_dkv, const float* __restrict__ inv_freq, T* __restrict__ q_pad, T* __restrict__ k_rows,
                       T* __restrict__ v_rows, const int* __restrict__ tok_pos, const int* __restrict__ kv_seq,
                       const int* __restrict__ kv_pos, const int* __restrict__ seq_page0, int n_q, int n_kv, int H, int d,
                       int p, int e, int r, int HD, int HDV, int page_size, const T* __restrict__ cache,
                       const int* __restrict__ seq_slot, const int* __restrict__ page_table, int pt_stride, int vec8) {
  // vec8: rows are moved in 16-byte pieces (bfloat16; d, p, e, HD, HDV, ld_kvx multiples of 8 and 16-byte aligned bases)
  extern __shared__ float sh[];     // cos [p/2], sin [p/2], rotated shared key part [p]
  zk_let_next_start();
  zk_wait_prior();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int half = p >> 1;
  float* cs = sh;
  float* sn = sh + half;
  float* kr = sh + p;
  const T zero = from_f32<T>(0.f);
  if (blockIdx.y == 0) {
    if (t >= n_q) return;
    const int pos = tok_pos[t];
    for (int i = tid; i < half; i += LAT_THREADS) {
      const float ang = (float)pos * inv_freq[i];
      cs[i] = cosf(ang);
      sn[i] = sinf(ang);
    }
    __syncthreads();
    if (sizeof(T) == 2 && vec8) {        // whole 16-byte pieces: a piece lies in one of the three parts of a row
      const int CH = HD / 8;
      for (int idx = tid; idx < H * CH; idx += LAT_THREADS) {
        const int h = idx / CH, j0 = (idx - h * CH) * 8;
        const T* qh = q + ((size_t)t * H + h) * (d + p);
        uint4 piece = make_uint4(0u, 0u, 0u, 0u);
        if (j0 < d) {
          piece = *reinterpret_cast<const uint4*>(qh + j0);
        } else if (j0 < d + p) {
          __align__(16) T vals[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int i = j0 - d + u;
            vals[u] = i < half ? from_f32<T>(to_f32(qh[d + i]) * cs[i] - to_f32(qh[d + i + half]) * sn[i])
                               : from_f32<T>(to_f32(qh[d + i - half]) * sn[i - half] + to_f32(qh[d + i]) * cs[i - half]);
          }
          piece = *reinterpret_cast<const uint4*>(vals);
        }
        *reinterpret_cast<uint4*>(q_pad + ((size_t)t * H + h) * HD + j0) = piece;
      }
      return;
    }
    for (int idx = tid; idx < H * HD; idx += LAT_THREADS) {
      const int h = idx / HD, j = idx - h * HD;
      const T* qh = q + ((size_t)t * H + h) * (d + p);
      T qv = zero;
      if (j < d) {
        qv = qh[j];
      } else if (j < d + p) {
        const int i = j - d;
        if (i < half) qv = from_f32<T>(to_f32(qh[d + i]) * cs[i] - to_f32(qh[d + i + half]) * sn[i]);
        else qv = from_f32<T>(to_f32(qh[d + i - half]) * sn[i - half] + to_f32(qh[d + i]) * cs[i - half]);
      }
      q_pad[((size_t)t * H + h) * HD + j] = qv;
    }
    return;
  }
  if (t >= n_kv) return;
  const int pos = kv_pos[t], b = kv_seq[t];
  if (cache) {
    const int cpage = page_table[(size_t)seq_slot[b] * pt_stride + pos / page_size];
    const T* row = cache + ((size_t)(cpage < 0 ? 0 : cpage) * page_size + pos % page_size) * (r + p) + r;
    for (int i = tid; i < p; i += LAT_THREADS) kr[i] = cpage < 0 ? 0.f : to_f32(row[i]);
  } else {
    const float* src = dkv + (size_t)t * ld_dkv + r;
    for (int i = tid; i < half; i += LAT_THREADS) {
      const float ang = (float)pos * inv_freq[i];
      const float c = cosf(ang), s = sinf(ang);
      const float u = src[i], v = src[i + half];
      kr[i] = u * c - v * s;
      kr[i + half] = u * s + v * c;
    }
  }
  __syncthreads();
  const size_t page = (size_t)seq_page0[b] + pos / page_size;
  const int in_page = pos % page_size;
  if (sizeof(T) == 2 && vec8) {
    const int CH = HD / 8, CHV = HDV / 8;
    for (int idx = tid; idx < H * CH; idx += LAT_THREADS) {
      const int h = idx / CH, j0 = (idx - h * CH) * 8;
      uint4 piece = make_uint4(0u, 0u, 0u, 0u);
      if (j0 < d) {
        piece = *reinterpret_cast<const uint4*>(kvx + (size_t)t * ld_kvx + (size_t)h * d + j0);
      } else if (j0 < d + p) {
        __align__(16) T vals[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) vals[u] = from_f32<T>(kr[j0 - d + u]);
        piece = *reinterpret_cast<const uint4*>(vals);
      }
      *reinterpret_cast<uint4*>(k_rows + ((page * H + h) * page_size + in_page) * HD + j0) = piece;
    }
    for (int idx = tid; idx < H * CHV; idx += LAT_THREADS) {
      const int h = idx / CHV, j0 = (idx - h * CHV) * 8;
      uint4 piece = make_uint4(0u, 0u, 0u, 0u);
      if (j0 < e) piece = *reinterpret_cast<const uint4*>(kvx + (size_t)t * ld_kvx + (size_t)H * d + (size_t)h * e + j0);
      *reinterpret_cast<uint4*>(v_rows + ((page * H + h) * page_size + in_page) * HDV + j0) = piece;
    }
    return;
  }
  for (int idx = tid; idx < H * HD; idx += LAT_THREADS) {
    const int h = idx / HD, j = idx - h * HD;
    T kv = zero;
    if (j < d) kv = kvx[(size_t)t * ld_kvx + (size_t)h * d + j];
    else if (j < d + p) kv = from_f32<T>(kr[j - d]);
    k_rows[((page * H + h) * page_size + in_page) * HD + j] = kv;
  }
  for (int idx = tid; idx < H * HDV; idx += LAT_THREADS) {
    const int h = idx / HDV, j = idx - h * HDV;
    v_rows[((page * H + h) * page_size + in_page) * HDV + j] =
        j < e ? kvx[(size_t)t * ld_kvx + (size_t)H * d + (size_t)h * e + j] : zero;
  }
}

// c_all[j, :] = the first r entries of the cache row of key/value token (kv_seq[j], kv_pos[j]); zeros for a page
// that is not there.  One block per token.
template <typename T>
__global__ void __launch_bounds__(LAT_THREADS)
    latent_gather_kernel(const T* __restrict__ cache, T* __restrict__ c_all, const int* __restrict__ kv_seq,
                         const int* __restrict__ kv_pos, const int* __restrict__ seq_slot,
                         const int* __restrict__ page_table, int pt_stride, int r, int W, int page_size) {
  zk_let_next_start();
  zk_wait_prior();
  const int j = blockIdx.x, pos = kv_pos[j];
  const int page = page_table[(size_t)seq_slot[kv_seq[j]] * pt_stride + pos / page_size];
  const T* row = cache + ((size_t)(page < 0 ? 0 : page) * page_size + pos % page_size) * W;
  for (int i = threadIdx.x; i < r; i += LAT_THREADS) c_all[(size_t)j * r + i] = page < 0 ? from_f32<T>(0.f) : row[i];
}

// out[t, h, n] = (sum_k a[t, h, k] * w[h, n, k]) * (gate ? sigmoid(gate[t * ld_gate + h]) : 1).
// a rows `lda` apart with head h at column h * a_head; out rows `ldo` apart with head h at column h * o_head;
// w [H, N, K] contiguous.  Block = (head, slice of N, group of LAT_ROWS tokens): the tokens' inputs wait in shared
// memory as float32, a warp owns an output column at a time and its lanes walk K, so every weight is read once per
// group of tokens and a sum's order depends on nothing but K.
#define LAT_ROWS 8
template <typename T>
__global__ void __launch_bounds__(LAT_THREADS)
    head_gemm_kernel(const T* __restrict__ a, int lda, int a_head, const T* __restrict__ w, T* __restrict__ out, int ldo,
                     int o_head, const float* __restrict__ gate, int ld_gate, int n, int N, int K, int cols_per_block) {
  extern __shared__ float as[];     // [LAT_ROWS][K]
  zk_let_next_start();
  zk_wait_prior();
  const int h = blockIdx.x, t0 = blockIdx.z * LAT_ROWS;
  const int rows = min(LAT_ROWS, n - t0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = LAT_THREADS / 32;
  for (int idx = threadIdx.x; idx < LAT_ROWS * K; idx += LAT_THREADS) {
    const int rr = idx / K, k = idx - rr * K;
    as[idx] = rr < rows ? to_f32(a[(size_t)(t0 + rr) * lda + (size_t)h * a_head + k]) : 0.f;
  }
  __syncthreads();
  const int c0 = blockIdx.y * cols_per_block, c1 = min(N, c0 + cols_per_block);
  for (int col = c0 + warp; col < c1; col += nw) {
    const T* wr = w + ((size_t)h * N + col) * K;
    float acc[LAT_ROWS];
#pragma unroll
    for (int rr = 0; rr < LAT_ROWS; ++rr) acc[rr] = 0.f;
    for (int k = lane; k < K; k += 32) {
      const float wv = to_f32(wr[k]);
#pragma unroll
      for (int rr = 0; rr < LAT_ROWS; ++rr) acc[rr] = fmaf(as[rr * K + k], wv, acc[rr]);
    }
#pragma unroll
    for (int rr = 0; rr < LAT_ROWS; ++rr) acc[rr] = warp_sum(acc[rr]);
    if (lane < rows) {
      float v = 0.f;
#pragma unroll
      for (int rr = 0; rr < LAT_ROWS; ++rr)
        if (lane == rr) v = acc[rr];
      if (gate) v = v / (1.0f + expf(-gate[(size_t)(t0 + lane) * ld_gate + h]));
      out[(size_t)(t0 + lane) * ldo + (size_t)h * o_head + col] = from_f32<T>(v);
    }
  }
}

extern "C" {

int zk_latent_prepare(const void* q, void* q_full, const float* dkv, int ld_dkv, const float* c_w, const float* inv_freq,
                      void* cache, const int* tok_seq, const int* tok_pos, const int* seq_slot, const int* page_table,
                      int pt_stride, int n_tokens, int H, int d, int p, int r, float eps, int page_size, int write_kv,
                      int dtype, int* status, void* c_out, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || d <= 0 || p <= 0 || (p & 1) || r <= 0 || page_size <= 0 || ld_dkv < r + p || !inv_freq || !c_w) return ZK_EINVAL;
  const dim3 grid(n_tokens, 2);
  if (dtype == ZK_F32)
    return zk_launch_dependent(latent_prepare_kernel<float>, grid, dim3(LAT_THREADS), 0, stream, (const float*)q, (float*)q_full,
                               dkv, ld_dkv, c_w, inv_freq, (float*)cache, tok_seq, tok_pos, seq_slot, page_table, pt_stride,
                               H, d, p, r, eps, page_size, write_kv, status, (float*)c_out);
  if (dtype == ZK_BF16)
    return zk_launch_dependent(latent_prepare_kernel<bf16>, grid, dim3(LAT_THREADS), 0, stream, (const bf16*)q, (bf16*)q_full,
                               dkv, ld_dkv, c_w, inv_freq, (bf16*)cache, tok_seq, tok_pos, seq_slot, page_table, pt_stride,
                               H, d, p, r, eps, page_size, write_kv, status, (bf16*)c_out);
  return ZK_EINVAL;
}

int zk_latent_pack(const void* q, const void* kvx, int ld_kvx, const float* dkv, int ld_dkv, const float* inv_freq,
                   void* q_pad, void* k_rows, void* v_rows, const int* tok_pos, const int* kv_seq, const int* kv_pos,
                   const int* seq_page0, int n_q, int n_kv, int H, int d, int p, int e, int r, int HD, int HDV,
                   int page_size, const void* cache, const int* seq_slot, const int* page_table, int pt_stride, int dtype,
                   cudaStream_t stream) {
  if (n_q <= 0 && n_kv <= 0) return 0;
  if (H <= 0 || d <= 0 || p <= 0 || (p & 1) || e <= 0 || r <= 0 || HD < d + p || HDV < e || page_size <= 0 ||
      ld_kvx < H * (d + e))
    return ZK_EINVAL;
  if (cache ? (!seq_slot || !page_table) : (!dkv || ld_dkv < r + p)) return ZK_EINVAL;
  const size_t smem = sizeof(float) * 2 * (size_t)p;
  if (smem > 48 * 1024) return ZK_EINVAL;
  const dim3 grid(n_q > n_kv ? n_q : n_kv, 2);
  const int vec8 = dtype == ZK_BF16 && !((d | p | e | HD | HDV | ld_kvx) & 7) &&
                   !(((uintptr_t)q | (uintptr_t)kvx | (uintptr_t)q_pad | (uintptr_t)k_rows | (uintptr_t)v_rows) & 15);
  if (dtype == ZK_F32)
    return zk_launch_dependent(latent_pack_kernel<float>, grid, dim3(LAT_THREADS), smem, stream, (const float*)q,
                               (const float*)kvx, ld_kvx, dkv, ld_dkv, inv_freq, (float*)q_pad, (float*)k_rows,
                               (float*)v_rows, tok_pos, kv_seq, kv_pos, seq_page0, n_q, n_kv, H, d, p, e, r, HD, HDV,
                               page_size, (const float*)cache, seq_slot, page_table, pt_stride, 0);
  if (dtype == ZK_BF16)
    return zk_launch_dependent(latent_pack_kernel<bf16>, grid, dim3(LAT_THREADS), smem, stream, (const bf16*)q,
                               (const bf16*)kvx, ld_kvx, dkv, ld_dkv, inv_freq, (bf16*)q_pad, (bf16*)k_rows,
                               (bf16*)v_rows, tok_pos, kv_seq, kv_pos, seq_page0, n_q, n_kv, H, d, p, e, r, HD, HDV,
                               page_size, (const bf16*)cache, seq_slot, page_table, pt_stride, vec8);
  return ZK_EINVAL;
}

// The latents of cached tokens, packed: c_all [n_kv, r] from cache [pages, 1, page_size, W].
int zk_latent_gather(const void* cache, void* c_all, const int* kv_seq, const int* kv_pos, const int* seq_slot,
                     const int* page_table, int pt_stride, int n_kv, int r, int W, int page_size, int dtype,
                     cudaStream_t stream) {
  if (n_kv <= 0) return 0;
  if (r <= 0 || W < r || page_size <= 0) return ZK_EINVAL;
  if (dtype == ZK_F32)
    return zk_launch_dependent(latent_gather_kernel<float>, dim3(n_kv), dim3(LAT_THREADS), 0, stream, (const float*)cache,
                               (float*)c_all, kv_seq, kv_pos, seq_slot, page_table, pt_stride, r, W, page_size);
  if (dtype == ZK_BF16)
    return zk_launch_dependent(latent_gather_kernel<bf16>, dim3(n_kv), dim3(LAT_THREADS), 0, stream, (const bf16*)cache,
                               (bf16*)c_all, kv_seq, kv_pos, seq_slot, page_table, pt_stride, r, W, page_size);
  return ZK_EINVAL;
}

int zk_head_gemm(const void* a, int lda, int a_head, const void* w, void* out, int ldo, int o_head, const float* gate,
                 int ld_gate, int n, int H, int N, int K, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (H <= 0 || N <= 0 || K <= 0 || lda < 0 || ldo < 0) return ZK_EINVAL;
  const size_t smem = sizeof(float) * LAT_ROWS * (size_t)K;
  if (smem > 200 * 1024) return ZK_EINVAL;
  const int groups = (n + LAT_ROWS - 1) / LAT_ROWS;
  int cols = N;                                    // enough blocks for the GPU when the tokens are few
  while (cols > 8 && (long long)H * groups * ((N + cols - 1) / cols) < 2 * 148) cols = (cols + 1) / 2;
  cols = (cols + 7) / 8 * 8;
  const dim3 grid(H, (N + cols - 1) / cols, groups);
  if (grid.y > 65535 || grid.z > 65535) return ZK_EINVAL;
#define ZK_HG(T)                                                                                                     \
  do {                                                                                                               \
    auto kern = head_gemm_kernel<T>;                                                                                 \
    if (smem > 48 * 1024) {                                                                                          \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
      if (e != cudaSuccess) return (int)e;                                                                           \
    }                                                                                                                \
    return zk_launch_dependent(kern, grid, dim3(LAT_THREADS), smem, stream, (const T*)a, lda, a_head, (const T*)w,   \
                               (T*)out, ldo, o_head, gate, ld_gate, n, N, K, cols);                                  \
  } while (0)
  if (dtype == ZK_F32) ZK_HG(float);
  if (dtype == ZK_BF16) ZK_HG(bf16);
#undef ZK_HG
  return ZK_EINVAL;
}

}  // extern "C"
