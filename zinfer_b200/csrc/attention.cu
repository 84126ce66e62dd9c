// Attention over the paged cache: (1) per-head q/k RMSNorm + rotary encoding + cache write,
// (2) causal grouped-query attention of a packed batch against the pages, with an optional
// window and an optional split of the keys into chunks, (3) the merge of the chunks.
//
// Softmax, norms and rotation angles are float32; the cache holds the run dtype.
// Cache layout of one layer: K and V are each [num_pages, kv_heads, page_size, head_dim];
// position p of a sequence lives in page page_table[slot][p / page_size] at row p % page_size.
//
// Reference: per-head norms and RoPE before the cache write, src/model.zig:1736-1773;
// NeoX pairing, src/rope.zig:50-64; angle = float(pos) * f_i, src/rope.zig:34-45; queries of one
// KV head ordered (token, head in group), src/model.zig:1352-1366; online softmax
// m, l, o with result o / l, src/attention.zig:478-517, 737-745; merge of split chunks,
// src/attention.zig:749-814.  No tile is skipped here (the reference drops tiles whose
// maximum is 13 below the running maximum, src/attention.zig:493).
#include "common.cuh"
#include <math.h>

#define ATT_MAX_HD 640
#define ATT_ROWS 16      // query rows (token, head-in-group) per block
#define ATT_TK 32        // keys per tile: one lane per key
#define ATT_WARPS 4

// ---------------------------------------------------------------------------------------
// (1) q/k norm + rope + cache write.  One warp per (token, head slot); head slots are the H
// query heads, then the Hkv key heads, then the Hkv value heads, as they lie in a qkv row.
// With `dense_out` the results of all three kinds go to a dense [n, (H + 2 Hkv) * hd] tensor
// instead (no cache write): the first half of a two-step path for position encodings that
// are not a rotation table.
__device__ __forceinline__ float query_temperature(int pos, float coef, int every) {
  return 1.0f + coef * logf((float)((pos + 1) / every + 1));
}

template <typename T>
__global__ void qk_prepare_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ dense_out,
                                  T* __restrict__ k_cache,
                                  T* __restrict__ v_cache, const float* __restrict__ q_w, const float* __restrict__ k_w,
                                  const float* __restrict__ inv_freq, const int* __restrict__ tok_seq,
                                  const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                                  const int* __restrict__ page_table, int pt_stride, int n_tokens, int H, int Hkv,
                                  int hd, int n_rot, int interleaved, float eps, int page_size, int write_kv,
                                  int* status, int vd, int unit_norm_after, float qt_coef, int qt_every) {
  // vd: width of a value head (a row of qkv is [q H*hd | k Hkv*hd | v Hkv*vd]).  unit_norm_after: q and k
  // heads are divided by their root mean square (no weight) AFTER the rotation; q_w / k_w, if given,
  // weigh an RMS norm BEFORE it.  qt_every > 0: a query at position p is multiplied, last of all, by
  // 1 + qt_coef * ln(floor((p + 1) / qt_every) + 1) (a temperature that grows with the position), in float32.
  __shared__ float sm_all[ATT_WARPS][ATT_MAX_HD];
  zk_wait_prior();   // nothing of the kernels before is read, and nothing written, above this line
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slots = H + 2 * Hkv;
  const long long item = (long long)blockIdx.x * ATT_WARPS + warp;
  if (item >= (long long)n_tokens * slots) return;
  const int t = (int)(item / slots), s = (int)(item % slots);
  const int kind = s < H ? 0 : (s < H + Hkv ? 1 : 2);  // 0 q, 1 k, 2 v
  if (kind != 0 && !write_kv && !dense_out) return;
  float* sm = sm_all[warp];
  const size_t row_w = (size_t)(H + Hkv) * hd + (size_t)Hkv * vd;
  const int wd = kind == 2 ? vd : hd;
  const size_t col0 = kind == 2 ? (size_t)(H + Hkv) * hd + (size_t)(s - H - Hkv) * vd : (size_t)s * hd;
  const T* src = qkv + (size_t)t * row_w + col0;
  const float* w = kind == 0 ? q_w : (kind == 1 ? k_w : nullptr);

  float ss = 0.f;
  for (int d = lane; d < wd; d += 32) {
    const float v = to_f32(src[d]);
    sm[d] = v;
    ss = fmaf(v, v, ss);
  }
  if (w) {
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)hd + eps);
    for (int d = lane; d < hd; d += 32) sm[d] = (sm[d] * scale) * w[d];
  }
  __syncwarp();
  const int pos = tok_pos[t];
  if (kind != 2 && inv_freq) {
    const int half = n_rot >> 1;
    for (int i = lane; i < half; i += 32) {
      const int ia = interleaved ? 2 * i : i;
      const int ib = interleaved ? 2 * i + 1 : i + half;
      const float ang = (float)pos * inv_freq[i];
      const float c = cosf(ang), sn = sinf(ang);
      const float a = sm[ia], b = sm[ib];
      sm[ia] = a * c - b * sn;
      sm[ib] = a * sn + b * c;
    }
    __syncwarp();
  }
  if (kind != 2 && unit_norm_after) {
    float s2 = 0.f;
    for (int d = lane; d < hd; d += 32) s2 = fmaf(sm[d], sm[d], s2);
    s2 = warp_sum(s2);
    const float scale = 1.0f / sqrtf(s2 / (float)hd + eps);
    for (int d = lane; d < hd; d += 32) sm[d] *= scale;
    __syncwarp();
  }
  if (kind == 0 && qt_every > 0) {
    const float temp = query_temperature(pos, qt_coef, qt_every);
    for (int d = lane; d < hd; d += 32) sm[d] *= temp;
    __syncwarp();
  }
  T* dst;
  if (dense_out) {
    dst = dense_out + (size_t)t * row_w + col0;
  } else if (kind == 0) {
    dst = q_out + (size_t)t * H * hd + (size_t)s * hd;
  } else {
    const int slot = seq_slot[tok_seq[t]];
    const int page = page_table[(size_t)slot * pt_stride + pos / page_size];
    if (page < 0) {
      if (lane == 0) atomicExch(status, 2);
      return;
    }
    const int kh = kind == 1 ? s - H : s - H - Hkv;
    T* base = kind == 1 ? k_cache : v_cache;
    dst = base + (((size_t)page * Hkv + kh) * page_size + pos % page_size) * wd;
  }
  for (int d = lane; d < wd; d += 32) dst[d] = from_f32<T>(sm[d]);
}

// The same for prompt steps with head sizes 64 and 128 and a rotation over the whole head in
// half-split pairing (or none): one block per token, its warps take the head slots in turn, the
// angles' cosines and sines are computed once per warp instead of once per head, and a lane keeps
// its pairs (d, d + hd/2) in registers.  The arithmetic and its order are those of
// qk_prepare_kernel, so both give the same bits.
template <typename T, int HD>
__global__ void __launch_bounds__(ATT_WARPS * 32)
    qk_prepare_token_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_cache,
                            T* __restrict__ v_cache, const float* __restrict__ q_w, const float* __restrict__ k_w,
                            const float* __restrict__ inv_freq, const int* __restrict__ tok_seq,
                            const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                            const int* __restrict__ page_table, int pt_stride, int H, int Hkv, float eps, int page_size,
                            int write_kv, int* status, float qt_coef, int qt_every) {
  constexpr int E = HD / 64, HALF = HD / 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;
  const int slots = H + 2 * Hkv;
  zk_let_next_start();
  zk_wait_prior();   // qkv is the kernel before's result
  const int pos = tok_pos[t];
  float cs[E], sn[E];
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const float ang = inv_freq ? (float)pos * inv_freq[lane + 32 * e] : 0.f;
    cs[e] = cosf(ang);
    sn[e] = sinf(ang);
  }
  const float temp = qt_every > 0 ? query_temperature(pos, qt_coef, qt_every) : 1.0f;
  int page = -2;   // not looked up yet
  const int n_slots = write_kv ? slots : H;
  // A warp's head slots four at a time: their loads are all under way before the first is used.
  // One after the other, a warp waited for memory once per slot, and the kernel's time was that
  // chain (18 us for 2,048 tokens of 48 slots, whose 25 MB would take 5).
  constexpr int UN = 4;
  for (int s0 = warp; s0 < n_slots; s0 += ATT_WARPS * UN) {
    float av[UN][E], bv[UN][E];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int s = s0 + u * ATT_WARPS;
      const T* src = qkv + (size_t)t * slots * HD + (size_t)min(s, n_slots - 1) * HD;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        av[u][e] = to_f32(src[lane + 32 * e]);
        bv[u][e] = to_f32(src[lane + 32 * e + HALF]);
      }
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int s = s0 + u * ATT_WARPS;
      if (s >= n_slots) break;
      const int kind = s < H ? 0 : (s < H + Hkv ? 1 : 2);
      const float* w = kind == 0 ? q_w : (kind == 1 ? k_w : nullptr);
      float a[E], b[E];
#pragma unroll
      for (int e = 0; e < E; ++e) {
        a[e] = av[u][e];
        b[e] = bv[u][e];
      }
      if (w) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) ss = fmaf(a[e], a[e], ss);
#pragma unroll
        for (int e = 0; e < E; ++e) ss = fmaf(b[e], b[e], ss);
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          a[e] = (a[e] * scale) * w[lane + 32 * e];
          b[e] = (b[e] * scale) * w[lane + 32 * e + HALF];
        }
      }
      if (kind != 2 && inv_freq) {
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float x = a[e], y = b[e];
          a[e] = x * cs[e] - y * sn[e];
          b[e] = x * sn[e] + y * cs[e];
        }
      }
      T* dst;
      if (kind == 0) {
        if (qt_every > 0) {
#pragma unroll
          for (int e = 0; e < E; ++e) {
            a[e] *= temp;
            b[e] *= temp;
          }
        }
        dst = q_out + (size_t)t * H * HD + (size_t)s * HD;
      } else {
        if (page == -2) page = page_table[(size_t)seq_slot[tok_seq[t]] * pt_stride + pos / page_size];
        if (page < 0) {
          if (lane == 0) atomicExch(status, 2);
          continue;
        }
        const int kh = kind == 1 ? s - H : s - H - Hkv;
        dst = (kind == 1 ? k_cache : v_cache) + (((size_t)page * Hkv + kh) * page_size + pos % page_size) * HD;
      }
#pragma unroll
      for (int e = 0; e < E; ++e) {
        dst[lane + 32 * e] = from_f32<T>(a[e]);
        dst[lane + 32 * e + HALF] = from_f32<T>(b[e]);
      }
    }
  }
}

// The same step for a mixer whose q and k norms run over the WHOLE projection (all heads of a
// token at once, weight of that width) and whose values may have another width than its keys;
// no rotation.  A row of `qkv` holds [q (H * hd) | k (Hkv * hd) | v (Hkv * vd)], or q alone when
// the call reads another call's cache (write_kv = 0).  Sums of squares are float32 and added in an
// order that the thread layout alone fixes.
#define SPAN_THREADS 256
#define SPAN_KEEP 8       // values a thread keeps between the sum of squares and the scaling: rows of up to 2048

// RMSNorm of one row of n values over its whole width (weight w, or none), written through `put(d, value)`.
// Rows of up to SPAN_THREADS * SPAN_KEEP values are read once; the sum of squares is added per thread in
// the order of its values and over the block in the order of the threads.
template <typename T, typename Put>
__device__ __forceinline__ void span_norm_row(const T* __restrict__ row, int n, const float* __restrict__ w, float eps,
                                              float* scratch, Put put) {
  const int tid = threadIdx.x;
  float keep[SPAN_KEEP];
  const bool fits = n <= SPAN_THREADS * SPAN_KEEP;
  float ss = 0.f;
  if (fits) {
#pragma unroll
    for (int i = 0; i < SPAN_KEEP; ++i) {
      const int d = tid + i * SPAN_THREADS;
      keep[i] = d < n ? to_f32(row[d]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < SPAN_KEEP; ++i) ss = fmaf(keep[i], keep[i], ss);
  } else {
    for (int d = tid; d < n; d += SPAN_THREADS) {
      const float v = to_f32(row[d]);
      ss = fmaf(v, v, ss);
    }
  }
  float scale = 1.f;
  if (w) {
    ss = block_sum(ss, scratch);
    scale = 1.0f / sqrtf(ss / (float)n + eps);
  }
  if (fits) {
#pragma unroll
    for (int i = 0; i < SPAN_KEEP; ++i) {
      const int d = tid + i * SPAN_THREADS;
      if (d < n) put(d, w ? (keep[i] * scale) * w[d] : keep[i]);
    }
  } else {
    for (int d = tid; d < n; d += SPAN_THREADS) {
      const float v = to_f32(row[d]);
      put(d, w ? (v * scale) * w[d] : v);
    }
  }
}

// Element d of a row of heads (hd wide each) after the rotation of the first n_rot entries of every head, entry i
// paired with entry i + n_rot/2; `buf` holds the row before the rotation.
__device__ __forceinline__ float span_rotated(const float* __restrict__ buf, int d, int hd, int n_rot,
                                              const float* __restrict__ inv_freq, int pos) {
  const int e = d % hd;
  if (e >= n_rot) return buf[d];
  const int half = n_rot >> 1;
  const float ang = (float)pos * inv_freq[e < half ? e : e - half];
  const float c = cosf(ang), sn = sinf(ang);
  return e < half ? buf[d] * c - buf[d + half] * sn : buf[d - half] * sn + buf[d] * c;
}

// Block (t, 0) prepares the token's queries, block (t, 1) its keys and values (absent when write_kv = 0).
// With inv_freq the first n_rot entries of every q and k head are rotated by the token's position after the
// norm (pairs (i, i + n_rot/2)); the normalised row then waits in shared memory (max(H, Hkv) * hd floats).
template <typename T>
__global__ void __launch_bounds__(SPAN_THREADS)
    qk_prepare_span_kernel(const T* __restrict__ qkv, int ld, T* __restrict__ q_out, T* __restrict__ k_cache,
                           T* __restrict__ v_cache, const float* __restrict__ q_w, const float* __restrict__ k_w,
                           const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                           const int* __restrict__ seq_slot, const int* __restrict__ page_table, int pt_stride, int H,
                           int Hkv, int hd, int vd, float eps, int page_size, int* status,
                           const float* __restrict__ inv_freq, int n_rot) {
  __shared__ float scratch[32];
  extern __shared__ float span_row[];
  zk_let_next_start();
  zk_wait_prior();   // qkv is the kernel before's result
  const int t = blockIdx.x, tid = threadIdx.x;
  const int qd = H * hd, kd = Hkv * hd;
  const T* row = qkv + (size_t)t * ld;
  const int pos = tok_pos[t];
  if (blockIdx.y == 0) {
    T* dst = q_out + (size_t)t * qd;
    if (inv_freq) {
      span_norm_row(row, qd, q_w, eps, scratch, [&](int d, float v) { span_row[d] = v; });
      __syncthreads();
      for (int d = tid; d < qd; d += SPAN_THREADS) dst[d] = from_f32<T>(span_rotated(span_row, d, hd, n_rot, inv_freq, pos));
      return;
    }
    span_norm_row(row, qd, q_w, eps, scratch, [&](int d, float v) { dst[d] = from_f32<T>(v); });
    return;
  }
  const int page = page_table[(size_t)seq_slot[tok_seq[t]] * pt_stride + pos / page_size];
  if (page < 0) {
    if (tid == 0) atomicExch(status, 2);
    return;
  }
  const int in_page = pos % page_size;
  if (inv_freq) {
    span_norm_row(row + qd, kd, k_w, eps, scratch, [&](int d, float v) { span_row[d] = v; });
    __syncthreads();
    for (int d = tid; d < kd; d += SPAN_THREADS) {
      const int kh = d / hd, e = d - kh * hd;
      k_cache[(((size_t)page * Hkv + kh) * page_size + in_page) * hd + e] =
          from_f32<T>(span_rotated(span_row, d, hd, n_rot, inv_freq, pos));
    }
  } else {
    span_norm_row(row + qd, kd, k_w, eps, scratch, [&](int d, float v) {
      const int kh = d / hd, e = d - kh * hd;
      k_cache[(((size_t)page * Hkv + kh) * page_size + in_page) * hd + e] = from_f32<T>(v);
    });
  }
  const T* vrow = row + qd + kd;
  for (int d = tid; d < Hkv * vd; d += SPAN_THREADS) {
    const int kh = d / vd, e = d - kh * vd;
    v_cache[(((size_t)page * Hkv + kh) * page_size + in_page) * vd + e] = vrow[d];
  }
}

// ---------------------------------------------------------------------------------------
// (2) attention.  Block = (query tile, kv head x head chunk, key split).  A query tile is
// `bq` consecutive tokens of one sequence; its rows are (token, head in group) pairs, at
// most ATT_ROWS of them; row r belongs to warp r % 4.  Keys are walked in tiles of 32 that
// start at multiples of 32, one lane per key.
template <typename T, int NPL>
__global__ void __launch_bounds__(ATT_WARPS * 32)
    attn_fwd_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                    T* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                    const int* __restrict__ tile_seq, const int* __restrict__ tile_q0, const int* __restrict__ cu_q,
                    const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                    const int* __restrict__ page_table, int pt_stride, int n_tokens, int H, int Hkv, int hd,
                    int page_size, int window, float scale, int bq, int gc, int num_splits, int split_keys, int vd,
                    const float* __restrict__ bias_r1, const float* __restrict__ bias_r2, int cross, int keep,
                    const float* __restrict__ sink, int v_from_k, float softcap) {
  // softcap > 0: a scaled score s becomes softcap * tanh(s / softcap) before anything else is done with it.
  // keep: with a window, the first `keep` positions of a sequence stay visible to every later query.
  // sink [H]: exp(sink_h) is one more term of head h's softmax denominator (no key, no value, unscaled).
  // v_from_k: a value row is the first vd entries of the key row (one vector per token serves as both).
  // vd: width of a value row (the keys' width is hd); NPL covers vd.  bias_r1 / bias_r2 [H]: with both
  // given, r1_h * ln(1 + r2_h * (i - j)) is taken off the scaled score of query i and key j (float32).
  // cross: every query head's weights are applied to the values of EVERY key/value head, one value head
  // per block (blockIdx.y also counts them), and the unnormalised sums go to part_o / part_ml whatever
  // num_splits is, rows ordered (split, token, head, value head): what a mix of the heads' weights
  // after the softmax needs (attn_merge_talk_kernel).
  extern __shared__ float smem[];
  float* qs = smem;                               // [ATT_ROWS][hd]
  float* Ks = qs + ATT_ROWS * hd;                 // [ATT_TK][hd + 1]
  float* Vs = Ks + ATT_TK * (hd + 1);             // [ATT_TK][vd]; with v_from_k the key tile itself
  const int vs_n = v_from_k ? 0 : ATT_TK * vd, vs_ld = v_from_k ? hd + 1 : vd;
  long long* rowoff = reinterpret_cast<long long*>(Vs + vs_n + ((ATT_TK * (hd + 1) + vs_n) & 1));  // [2][ATT_TK], 8-byte aligned
  if (v_from_k) Vs = Ks;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = H / Hkv;
  const int chunks = (g + gc - 1) / gc;
  const int kvh = (blockIdx.y / chunks) % Hkv, chunk = blockIdx.y % chunks;
  const int VH = cross ? Hkv : 1;
  const int vh = cross ? blockIdx.y / (chunks * Hkv) : kvh;      // the key/value head whose values this block reads
  const int b = tile_seq[blockIdx.x], q0 = tile_q0[blockIdx.x];
  const int split = blockIdx.z;
  const int t_base = cu_q[b], Tq = cu_q[b + 1] - t_base;
  const int start = seq_start[b];
  const int slot = seq_slot[b];
  const int* pt = page_table + (size_t)slot * pt_stride;

  // rows of this warp: r = warp + 4*i
  int row_t[4], row_h[4], row_lo[4], row_hi[4];
  bool row_ok[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = warp + ATT_WARPS * i;
    const int tq = r / gc, hl = r % gc;
    row_ok[i] = (tq < bq) && (q0 + tq < Tq) && (chunk * gc + hl < g);
    row_t[i] = t_base + q0 + tq;
    row_h[i] = kvh * g + chunk * gc + hl;
    row_hi[i] = start + q0 + tq + 1;
    row_lo[i] = (window > 0 && row_hi[i] > window) ? row_hi[i] - window : 0;
  }
  float r1[4], r2[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    r1[i] = (bias_r1 && row_ok[i]) ? bias_r1[row_h[i]] : 0.f;
    r2[i] = (bias_r2 && row_ok[i]) ? bias_r2[row_h[i]] : 0.f;
  }
  const bool biased = bias_r1 != nullptr && bias_r2 != nullptr;

  // stage the query rows as float32
  for (int idx = tid; idx < ATT_ROWS * hd; idx += ATT_WARPS * 32) {
    const int r = idx / hd, d = idx - r * hd;
    const int tq = r / gc, hl = r % gc;
    const bool ok = (tq < bq) && (q0 + tq < Tq) && (chunk * gc + hl < g);
    qs[idx] = ok ? to_f32(q[(size_t)(t_base + q0 + tq) * H * hd + (size_t)(kvh * g + chunk * gc + hl) * hd + d]) : 0.f;
  }

  // key range of the block
  const int last_tq = min(q0 + bq, Tq) - 1;
  int k_end = start + last_tq + 1;
  int k_begin = 0;
  if (window > 0) {
    const int first_hi = start + q0 + 1;
    k_begin = first_hi > window ? first_hi - window : 0;
  }
  // the kept first tokens that lie below the window's reach: tiles [a_lo, a_hi), walked before the window's
  int a_lo = 0, a_hi = (keep > 0 && k_begin > 0) ? min(keep, k_begin) : 0;
  if (num_splits > 1) {
    k_begin = max(k_begin, split * split_keys);
    k_end = min(k_end, (split + 1) * split_keys);
    a_lo = split * split_keys;
    a_hi = min(a_hi, (split + 1) * split_keys);
  }
  k_begin = (k_begin / ATT_TK) * ATT_TK;
  a_hi = min(a_hi, k_begin);                      // a tile the window's walk reaches anyway is not walked twice

  float m[4], l[4], o[4][NPL];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < NPL; ++c) o[i][c] = 0.f;
  }
  const int split_lo = num_splits > 1 ? split * split_keys : 0;

  for (int phase = 0; phase < 2; ++phase)
  for (int kb = phase ? k_begin : a_lo; kb < (phase ? k_end : a_hi); kb += ATT_TK) {
    __syncthreads();  // previous tile fully consumed (and qs staged, first time)
    if (tid < ATT_TK) {
      const int kp = kb + tid;
      long long off = -1;
      if (kp < k_end) {
        const int page = pt[kp / page_size];
        if (page >= 0) off = ((long long)page * Hkv + kvh) * page_size + kp % page_size;   // row index; x hd or vd below
      }
      rowoff[tid] = off;
      rowoff[ATT_TK + tid] = off < 0 ? off : off + (long long)(vh - kvh) * page_size;      // the value row
    }
    __syncthreads();
    for (int idx = tid; idx < ATT_TK * hd; idx += ATT_WARPS * 32) {
      const int j = idx / hd, d = idx - j * hd;
      const long long off = rowoff[j];
      Ks[j * (hd + 1) + d] = off >= 0 ? to_f32(k_cache[off * hd + d]) : 0.f;
    }
    for (int idx = tid; idx < vs_n; idx += ATT_WARPS * 32) {
      const int j = idx / vd, d = idx - j * vd;
      const long long off = rowoff[ATT_TK + j];
      Vs[j * vd + d] = off >= 0 ? to_f32(v_cache[off * vd + d]) : 0.f;
    }
    __syncthreads();

    float s[4] = {0.f, 0.f, 0.f, 0.f};
    const float* kr = Ks + lane * (hd + 1);
    for (int d = 0; d < hd; ++d) {
      const float kd = kr[d];
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i] = fmaf(qs[(warp + ATT_WARPS * i) * hd + d], kd, s[i]);
    }
    const int kp = kb + lane;
    const bool key_ok = kp < k_end && kp >= split_lo && rowoff[lane] >= 0;
    float p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const bool ok = row_ok[i] && key_ok && (kp >= row_lo[i] || kp < keep) && kp < row_hi[i];
      float sc = -INFINITY;
      if (ok) {
        sc = s[i] * scale;
        if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
        if (biased) sc -= r1[i] * log1pf(r2[i] * (float)(row_hi[i] - 1 - kp));
      }
      const float mt = warp_max(sc);
      if (mt == -INFINITY) {  // no key of this tile is visible to this row
        p[i] = 0.f;
        continue;
      }
      const float m_new = fmaxf(m[i], mt);
      const float alpha = expf(m[i] - m_new);
      p[i] = ok ? expf(sc - m_new) : 0.f;
      l[i] = l[i] * alpha + warp_sum(p[i]);
      m[i] = m_new;
#pragma unroll
      for (int c = 0; c < NPL; ++c) o[i][c] *= alpha;
    }
    for (int j = 0; j < ATT_TK; ++j) {
      float vj[NPL];
#pragma unroll
      for (int c = 0; c < NPL; ++c) {
        const int d = lane + 32 * c;
        vj[c] = d < vd ? Vs[j * vs_ld + d] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float pj = __shfl_sync(0xffffffffu, p[i], j);
#pragma unroll
        for (int c = 0; c < NPL; ++c) o[i][c] = fmaf(pj, vj[c], o[i][c]);
      }
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (!row_ok[i]) continue;
    if (num_splits == 1 && !cross) {
      if (sink) {                                 // one more term of the denominator
        const float sk = sink[row_h[i]];
        const float m_fin = fmaxf(m[i], sk);
        const float alpha = m[i] == -INFINITY ? 0.f : expf(m[i] - m_fin);
        l[i] = l[i] * alpha + expf(sk - m_fin);
#pragma unroll
        for (int c = 0; c < NPL; ++c) o[i][c] *= alpha;
      }
      const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
      T* dst = out + (size_t)row_t[i] * H * vd + (size_t)row_h[i] * vd;
#pragma unroll
      for (int c = 0; c < NPL; ++c) {
        const int d = lane + 32 * c;
        if (d < vd) dst[d] = from_f32<T>(o[i][c] * inv);
      }
    } else {
      const size_t row = (((size_t)split * n_tokens + row_t[i]) * H + row_h[i]) * VH + (cross ? vh : 0);
      float* dst = part_o + row * vd;
#pragma unroll
      for (int c = 0; c < NPL; ++c) {
        const int d = lane + 32 * c;
        if (d < vd) dst[d] = o[i][c];
      }
      if (lane == 0) {
        part_ml[row * 2] = m[i];
        part_ml[row * 2 + 1] = l[i];
      }
    }
  }
}

// (3) merge: out = sum_s e^{m_s - M} o_s / sum_s e^{m_s - M} l_s.  One warp per (token, head).
// A lane holds the (m, l) of one chunk (32 chunks at a time), so that the loads of all chunks are
// under way together; the sums run over the chunks in ascending order whatever the timing.
// With `sink` [H] (rows ordered (token, head)): exp(sink_h) is one more term of the denominator.  Rows wider than
// 256 values are merged 256 columns at a time.
template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ part_o_all, const float* __restrict__ part_ml,
                                  T* __restrict__ out_all, int n_rows, int hd_all, int num_splits,
                                  const float* __restrict__ sink, int H) {
  zk_let_next_start();
  zk_wait_prior();   // nothing of the kernels before is read, and nothing written, above this line
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  float M = sink ? sink[row % H] : -INFINITY;
  for (int s0 = 0; s0 < num_splits; s0 += 32) {
    const int s = s0 + lane;
    const float ms = s < num_splits ? part_ml[((size_t)s * n_rows + row) * 2] : -INFINITY;
    M = fmaxf(M, warp_max(ms));
  }
  for (int c0 = 0; c0 < hd_all; c0 += 256) {
  const int hd = min(256, hd_all - c0);
  const float* part_o = part_o_all + c0;
  T* out = out_all + c0;
  float L = sink ? expf(sink[row % H] - M) : 0.f;
  float acc[8];   // head sizes up to 256: 8 values per lane
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int s0 = 0; s0 < num_splits; s0 += 32) {
    const int s = s0 + lane;
    float ms = -INFINITY, ls = 0.f;
    if (s < num_splits) {
      const float2 ml = *reinterpret_cast<const float2*>(part_ml + ((size_t)s * n_rows + row) * 2);
      ms = ml.x;
      ls = ml.y;
    }
    const float e = ms == -INFINITY ? 0.f : expf(ms - M);
    const int n_here = min(32, num_splits - s0);
    for (int j = 0; j < n_here; ++j) L = fmaf(__shfl_sync(0xffffffffu, e, j), __shfl_sync(0xffffffffu, ls, j), L);
    for (int j0 = 0; j0 < n_here; j0 += 8) {
      float v[8][8], w[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int j = j0 + u;
        w[u] = j < n_here ? __shfl_sync(0xffffffffu, e, j & 31) : 0.f;
        const float* po = part_o + ((size_t)(s0 + j) * n_rows + row) * hd_all;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[u][i] = (w[u] != 0.f && lane + 32 * i < hd) ? po[lane + 32 * i] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[u], v[u][i], acc[i]);
    }
  }
  const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (lane + 32 * i < hd) out[(size_t)row * hd_all + lane + 32 * i] = from_f32<T>(acc[i] * inv);
  }
}

// (3b) merge for weights that are mixed across the heads after the softmax: with w_g(i, j) head g's softmax
// weights and T [H, H],   out[t, h, :] = sum_g T[h, g] * (sum_j w_g(t, j) v_{kv(h)}(j, :)).
// The inner sums are what the cross mode of attn_fwd_kernel left unnormalised per (split, token, head g,
// value head): merged over the splits as in attn_merge_kernel, then weighed and added in the order of g.
// One warp per (token, head h); float32 until the store.
template <typename T>
__global__ void attn_merge_talk_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       const float* __restrict__ talk, T* __restrict__ out, int n_tokens, int H, int Hkv,
                                       int vd, int num_splits) {
  zk_let_next_start();
  zk_wait_prior();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)n_tokens * H) return;
  const int t = (int)(item / H), h = (int)(item % H);
  const int c = h / (H / Hkv);
  const size_t rows_per_split = (size_t)n_tokens * H * Hkv;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int g = 0; g < H; ++g) {
    const size_t row = ((size_t)t * H + g) * Hkv + c;
    float M = -INFINITY;
    for (int s = 0; s < num_splits; ++s) M = fmaxf(M, part_ml[((size_t)s * rows_per_split + row) * 2]);
    float L = 0.f, og[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) og[i] = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const size_t r = (size_t)s * rows_per_split + row;
      const float ms = part_ml[r * 2];
      if (ms == -INFINITY) continue;
      const float e = expf(ms - M);
      L = fmaf(e, part_ml[r * 2 + 1], L);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (lane + 32 * i < vd) og[i] = fmaf(e, part_o[r * vd + lane + 32 * i], og[i]);
    }
    const float wgt = L > 0.f ? talk[h * H + g] / L : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(wgt, og[i], acc[i]);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (lane + 32 * i < vd) out[((size_t)t * H + h) * vd + lane + 32 * i] = from_f32<T>(acc[i]);
}

// The same with one block per (token, key/value head c): the H sums of that value head, merged over the splits
// and normalised, are first laid down in shared memory (a warp per row, the splits in ascending order), then
// every output value of the heads that belong to c adds its H terms in the order of g.  Each partial sum is
// read once, in whole lines.
template <typename T>
__global__ void __launch_bounds__(256)
    attn_merge_talk_token_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                 const float* __restrict__ talk, T* __restrict__ out, int n_tokens, int H, int Hkv, int vd,
                                 int num_splits) {
  extern __shared__ float mt_smem[];
  float* A = mt_smem;                      // [H][vd]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  const int per = H / Hkv;
  const int t = blockIdx.x, c = blockIdx.y;
  float* Tm = A + (size_t)H * vd;          // [per][H]: the rows of `talk` of this block's heads
  for (int i = tid; i < per * H; i += blockDim.x) Tm[i] = talk[(size_t)c * per * H + i];
  zk_let_next_start();
  zk_wait_prior();
  const size_t rows_per_split = (size_t)n_tokens * H * Hkv;
  for (int g = warp; g < H; g += nw) {
    const size_t row = ((size_t)t * H + g) * Hkv + c;
    float M = -INFINITY;
    for (int s = 0; s < num_splits; ++s) M = fmaxf(M, part_ml[((size_t)s * rows_per_split + row) * 2]);
    float L = 0.f, og[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) og[i] = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const size_t rr = (size_t)s * rows_per_split + row;
      const float ms = part_ml[rr * 2];
      if (ms == -INFINITY) continue;
      const float e = expf(ms - M);
      L = fmaf(e, part_ml[rr * 2 + 1], L);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (lane + 32 * i < vd) og[i] = fmaf(e, part_o[rr * vd + lane + 32 * i], og[i]);
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (lane + 32 * i < vd) A[(size_t)g * vd + lane + 32 * i] = og[i] * inv;
  }
  __syncthreads();
  for (int idx = tid; idx < per * vd; idx += blockDim.x) {
    const int hl = idx / vd, d = idx - hl * vd;
    float acc = 0.f;
    for (int g = 0; g < H; ++g) acc = fmaf(Tm[hl * H + g], A[(size_t)g * vd + d], acc);
    out[((size_t)t * H + c * per + hl) * vd + d] = from_f32<T>(acc);
  }
}

namespace {

size_t attn_smem_bytes(int hd, int vd) {     // vd = 0: the values are read from the key tile
  return sizeof(float) * ((size_t)ATT_ROWS * hd + (size_t)ATT_TK * (hd + 1) + (size_t)ATT_TK * vd + 1) + sizeof(long long) * 2 * ATT_TK + 16;
}

template <typename T, int NPL>
int launch_attn(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o, float* part_ml,
                const int* tile_seq, const int* tile_q0, const int* cu_q, const int* seq_start, const int* seq_slot,
                const int* page_table, int pt_stride, int n_tiles, int n_tokens, int H, int Hkv, int hd, int page_size,
                int window, float scale, int bq, int gc, int num_splits, int split_keys, int vd, const float* r1,
                const float* r2, int cross, int keep, const float* sink, int v_from_k, float softcap, cudaStream_t stream) {
  const size_t smem = attn_smem_bytes(hd, v_from_k ? 0 : vd);
  if (smem > 227 * 1024) return ZK_EINVAL;
  auto kern = attn_fwd_kernel<T, NPL>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int g = H / Hkv;
  const int chunks = (g + gc - 1) / gc;
  dim3 grid(n_tiles, Hkv * chunks * (cross ? Hkv : 1), num_splits);
  kern<<<grid, ATT_WARPS * 32, smem, stream>>>((const T*)q, (const T*)k_cache, (const T*)v_cache, (T*)out, part_o,
                                               part_ml, tile_seq, tile_q0, cu_q, seq_start, seq_slot, page_table,
                                               pt_stride, n_tokens, H, Hkv, hd, page_size, window, scale, bq, gc,
                                               num_splits, split_keys, vd, r1, r2, cross, keep, sink, v_from_k, softcap);
  return ZK_LAUNCH_STATUS();
}

template <typename T>
int dispatch_attn(int hd, const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o,
                  float* part_ml, const int* tile_seq, const int* tile_q0, const int* cu_q, const int* seq_start,
                  const int* seq_slot, const int* page_table, int pt_stride, int n_tiles, int n_tokens, int H, int Hkv,
                  int page_size, int window, float scale, int bq, int gc, int num_splits, int split_keys, int vd,
                  const float* r1, const float* r2, int cross, int keep, const float* sink, int v_from_k, float softcap,
                  cudaStream_t stream) {
#define ZK_ATT_CASE(N)                                                                                               \
  case N:                                                                                                            \
    return launch_attn<T, N>(q, k_cache, v_cache, out, part_o, part_ml, tile_seq, tile_q0, cu_q, seq_start, seq_slot, \
                             page_table, pt_stride, n_tiles, n_tokens, H, Hkv, hd, page_size, window, scale, bq, gc,  \
                             num_splits, split_keys, vd, r1, r2, cross, keep, sink, v_from_k, softcap, stream);
  int npl = (vd + 31) / 32;                 // value columns per lane: every count up to 8, then 12, 16, 20
  if (npl > 8) npl = npl <= 12 ? 12 : (npl <= 16 ? 16 : 20);
  switch (npl) {
    ZK_ATT_CASE(1) ZK_ATT_CASE(2) ZK_ATT_CASE(3) ZK_ATT_CASE(4) ZK_ATT_CASE(5) ZK_ATT_CASE(6) ZK_ATT_CASE(7)
    ZK_ATT_CASE(8) ZK_ATT_CASE(12) ZK_ATT_CASE(16) ZK_ATT_CASE(20)
  }
#undef ZK_ATT_CASE
  return ZK_EINVAL;
}

}  // namespace

extern "C" {

// Rows per block and the split of a KV group's heads, for the host to build its tile table:
// gc heads of a group per block, bq = ATT_ROWS / gc tokens per tile.
int zk_attn_rows_per_block() { return ATT_ROWS; }
int zk_attn_max_head_dim() { return ATT_MAX_HD; }

int zk_qk_prepare(const void* qkv, void* q_out, void* dense_out, void* k_cache, void* v_cache, const float* q_w, const float* k_w,
                  const float* inv_freq, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                  const int* page_table, int pt_stride, int n_tokens, int H, int Hkv, int hd, int n_rot,
                  int interleaved, float eps, int page_size, int write_kv, int dtype, int* status, int vd,
                  int unit_norm_after, float qt_coef, int qt_every, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hd <= 0 || hd > ATT_MAX_HD || H <= 0 || Hkv <= 0 || n_rot > hd || (n_rot & 1) || page_size <= 0) return ZK_EINVAL;
  if (vd <= 0) vd = hd;
  if (vd > ATT_MAX_HD) return ZK_EINVAL;
  // many tokens, whole-head half-split rotation (or none): one block per token
  if (n_tokens >= 256 && !dense_out && (hd == 64 || hd == 128) && vd == hd && !unit_norm_after &&
      (!inv_freq || (n_rot == hd && !interleaved)) &&
      (dtype == ZK_F32 || dtype == ZK_BF16)) {
#define ZK_QKP(T, HDV)                                                                                               \
  zk_launch_dependent(qk_prepare_token_kernel<T, HDV>, dim3(n_tokens), dim3(ATT_WARPS * 32), 0, stream,             \
      (const T*)qkv, (T*)q_out, (T*)k_cache, (T*)v_cache, q_w, k_w, inv_freq, tok_seq, tok_pos, seq_slot, page_table, \
      pt_stride, H, Hkv, eps, page_size, write_kv, status, qt_coef, qt_every)
    if (dtype == ZK_F32 && hd == 64) ZK_QKP(float, 64);
    else if (dtype == ZK_F32) ZK_QKP(float, 128);
    else if (hd == 64) ZK_QKP(bf16, 64);
    else ZK_QKP(bf16, 128);
#undef ZK_QKP
    return ZK_LAUNCH_STATUS();
  }
  const long long items = (long long)n_tokens * (H + 2 * Hkv);
  const int blocks = (int)((items + ATT_WARPS - 1) / ATT_WARPS);
  if (dtype == ZK_F32)
    return zk_launch_dependent(qk_prepare_kernel<float>, dim3(blocks), dim3(ATT_WARPS * 32), 0, stream,
        (const float*)qkv, (float*)q_out, (float*)dense_out, (float*)k_cache, (float*)v_cache, q_w, k_w, inv_freq, tok_seq, tok_pos,
        seq_slot, page_table, pt_stride, n_tokens, H, Hkv, hd, n_rot, interleaved, eps, page_size, write_kv, status, vd,
        unit_norm_after, qt_coef, qt_every);
  else if (dtype == ZK_BF16)
    return zk_launch_dependent(qk_prepare_kernel<bf16>, dim3(blocks), dim3(ATT_WARPS * 32), 0, stream,
        (const bf16*)qkv, (bf16*)q_out, (bf16*)dense_out, (bf16*)k_cache, (bf16*)v_cache, q_w, k_w, inv_freq, tok_seq, tok_pos, seq_slot,
        page_table, pt_stride, n_tokens, H, Hkv, hd, n_rot, interleaved, eps, page_size, write_kv, status, vd,
        unit_norm_after, qt_coef, qt_every);
  else
    return ZK_EINVAL;
  return ZK_LAUNCH_STATUS();
}

// q/k RMSNorm over the whole projection (weights [H*hd] and [Hkv*hd], either may be null), values vd wide.
// qkv rows are `ld` elements apart and hold q alone when write_kv = 0.
int zk_qk_prepare_span(const void* qkv, int ld, void* q_out, void* k_cache, void* v_cache, const float* q_w,
                       const float* k_w, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                       const int* page_table, int pt_stride, int n_tokens, int H, int Hkv, int hd, int vd, float eps,
                       int page_size, int write_kv, int dtype, int* status, const float* inv_freq, int n_rot,
                       cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hd <= 0 || vd <= 0 || H <= 0 || Hkv <= 0 || page_size <= 0) return ZK_EINVAL;
  if (ld < H * hd + (write_kv ? Hkv * (hd + vd) : 0)) return ZK_EINVAL;
  if (inv_freq && (n_rot <= 0 || (n_rot & 1) || n_rot > hd)) return ZK_EINVAL;
  const size_t smem = inv_freq ? sizeof(float) * (size_t)(H > Hkv ? H : Hkv) * hd : 0;
  if (smem > 160 * 1024) return ZK_EINVAL;
  if (dtype == ZK_F32) {
    auto kern = qk_prepare_span_kernel<float>;
    if (smem > 40 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    return zk_launch_dependent(kern, dim3(n_tokens, write_kv ? 2 : 1), dim3(SPAN_THREADS), smem, stream,
        (const float*)qkv, ld, (float*)q_out, (float*)k_cache, (float*)v_cache, q_w, k_w, tok_seq, tok_pos, seq_slot,
        page_table, pt_stride, H, Hkv, hd, vd, eps, page_size, status, inv_freq, n_rot);
  }
  if (dtype == ZK_BF16) {
    auto kern = qk_prepare_span_kernel<bf16>;
    if (smem > 40 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    return zk_launch_dependent(kern, dim3(n_tokens, write_kv ? 2 : 1), dim3(SPAN_THREADS), smem, stream,
        (const bf16*)qkv, ld, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, q_w, k_w, tok_seq, tok_pos, seq_slot,
        page_table, pt_stride, H, Hkv, hd, vd, eps, page_size, status, inv_freq, n_rot);
  }
  return ZK_EINVAL;
}

// q [n_tokens, H*hd], out [n_tokens, H*vd]; part_o [num_splits, n_tokens*H, hd] and part_ml [num_splits,
// n_tokens*H, 2] float32 scratch, used when num_splits > 1 (then call zk_attn_merge).
int zk_attn_fwd(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o, float* part_ml,
                const int* tile_seq, const int* tile_q0, const int* cu_q, const int* seq_start, const int* seq_slot,
                const int* page_table, int pt_stride, int n_tiles, int n_tokens, int H, int Hkv, int hd, int page_size,
                int window, float scale, int bq, int gc, int num_splits, int split_keys, int dtype, int vd,
                const float* bias_r1, const float* bias_r2, int cross, int keep, const float* sink, int v_from_k,
                float softcap, cudaStream_t stream) {
  if (n_tiles <= 0 || n_tokens <= 0) return 0;
  if (keep < 0 || (v_from_k && (vd > hd || cross))) return ZK_EINVAL;
  if (cross && (!part_o || !part_ml)) return ZK_EINVAL;
  if (hd <= 0 || hd > ATT_MAX_HD || H <= 0 || Hkv <= 0 || H % Hkv || page_size <= 0) return ZK_EINVAL;
  if (vd <= 0 || vd > ATT_MAX_HD || ((bias_r1 == nullptr) != (bias_r2 == nullptr))) return ZK_EINVAL;
  if (gc <= 0 || gc > ATT_ROWS || bq <= 0 || bq * gc > ATT_ROWS || num_splits < 1) return ZK_EINVAL;
  if (num_splits > 1 && (split_keys <= 0 || split_keys % ATT_TK || !part_o || !part_ml)) return ZK_EINVAL;
  if (dtype == ZK_F32)
    return dispatch_attn<float>(hd, q, k_cache, v_cache, out, part_o, part_ml, tile_seq, tile_q0, cu_q, seq_start,
                                seq_slot, page_table, pt_stride, n_tiles, n_tokens, H, Hkv, page_size, window, scale,
                                bq, gc, num_splits, split_keys, vd, bias_r1, bias_r2, cross, keep, sink, v_from_k, softcap, stream);
  if (dtype == ZK_BF16)
    return dispatch_attn<bf16>(hd, q, k_cache, v_cache, out, part_o, part_ml, tile_seq, tile_q0, cu_q, seq_start,
                               seq_slot, page_table, pt_stride, n_tiles, n_tokens, H, Hkv, page_size, window, scale, bq,
                               gc, num_splits, split_keys, vd, bias_r1, bias_r2, cross, keep, sink, v_from_k, softcap, stream);
  return ZK_EINVAL;
}

// part_o [num_splits, n_tokens*H*Hkv, vd], part_ml [num_splits, n_tokens*H*Hkv, 2] as the cross mode of zk_attn_fwd
// leaves them; talk float32 [H, H]; out [n_tokens, H*vd].
int zk_attn_merge_talk(const float* part_o, const float* part_ml, const float* talk, void* out, int n_tokens, int H, int Hkv,
                       int vd, int num_splits, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || Hkv <= 0 || H % Hkv || vd <= 0 || vd > ATT_MAX_HD || num_splits < 1 || !talk) return ZK_EINVAL;
  const size_t smem = ((size_t)H * vd + (size_t)(H / Hkv) * H) * sizeof(float);
  if (smem <= 200 * 1024 && Hkv <= 65535 && (dtype == ZK_F32 || dtype == ZK_BF16)) {
    if (dtype == ZK_F32) {
      auto kern = attn_merge_talk_token_kernel<float>;
      if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
      }
      return zk_launch_dependent(kern, dim3(n_tokens, Hkv), dim3(256), smem, stream, part_o, part_ml, talk, (float*)out, n_tokens,
                                 H, Hkv, vd, num_splits);
    }
    auto kern = attn_merge_talk_token_kernel<bf16>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    return zk_launch_dependent(kern, dim3(n_tokens, Hkv), dim3(256), smem, stream, part_o, part_ml, talk, (bf16*)out, n_tokens, H,
                               Hkv, vd, num_splits);
  }
  const int warps = 4;
  const long long items = (long long)n_tokens * H;
  const int blocks = (int)((items + warps - 1) / warps);
  if (dtype == ZK_F32)
    return zk_launch_dependent(attn_merge_talk_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, part_o, part_ml, talk,
                               (float*)out, n_tokens, H, Hkv, vd, num_splits);
  if (dtype == ZK_BF16)
    return zk_launch_dependent(attn_merge_talk_kernel<bf16>, dim3(blocks), dim3(warps * 32), 0, stream, part_o, part_ml, talk,
                               (bf16*)out, n_tokens, H, Hkv, vd, num_splits);
  return ZK_EINVAL;
}

int zk_attn_merge(const float* part_o, const float* part_ml, void* out, int n_rows, int hd, int num_splits, int dtype,
                  const float* sink, int H, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (sink && (H <= 0 || n_rows % H)) return ZK_EINVAL;
  const int warps = 4;
  const int blocks = (n_rows + warps - 1) / warps;
  if (dtype == ZK_F32)
    return zk_launch_dependent(attn_merge_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, part_o, part_ml, (float*)out, n_rows, hd, num_splits, sink, H);
  else if (dtype == ZK_BF16)
    return zk_launch_dependent(attn_merge_kernel<bf16>, dim3(blocks), dim3(warps * 32), 0, stream, part_o, part_ml, (bf16*)out, n_rows, hd, num_splits, sink, H);
  else
    return ZK_EINVAL;
  return ZK_LAUNCH_STATUS();
}

}  // extern "C"
