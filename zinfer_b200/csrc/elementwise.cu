// Row-wise kernels: embedding gather, RMSNorm (with optional row gather), SiLU-gate product.
// All arithmetic is float32; only loads and stores use the run dtype.
#include "common.cuh"
#include <stdint.h>

// x[t, :] = float(table[tokens[t], :]).  A token id outside [0, vocab) sets *status = 1 and
// yields a zero row (reference: row lookup of token_embd, src/model.zig:2352-2358).
// With `pos_table` [max_pos, dim] a learned position vector is added, unscaled, in float32:
// x[t, :] += float(pos_table[tok_pos[t], :]); a position outside the table sets *status = 3.
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table, float* __restrict__ x,
                             int dim, int vocab, float scale, int* status, const T* __restrict__ pos_table,
                             const int* __restrict__ tok_pos, int max_pos) {
  zk_let_next_start();
  zk_wait_prior();   // nothing of the kernels before is read, and nothing written, above this line
  const int t = blockIdx.x;
  const int tok = tokens[t];
  const bool ok = tok >= 0 && tok < vocab;
  if (!ok && threadIdx.x == 0) atomicExch(status, 1);
  const T* row = table + (size_t)(ok ? tok : 0) * dim;
  float* out = x + (size_t)t * dim;
  const T* prow = nullptr;
  if (pos_table) {
    const int p = tok_pos[t];
    if (p >= 0 && p < max_pos) prow = pos_table + (size_t)p * dim;
    else if (threadIdx.x == 0) atomicExch(status, 3);
  }
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float v = ok ? to_f32(row[d]) * scale : 0.f;
    if (prow) v += to_f32(prow[d]);
    out[d] = v;
  }
}

// y[r, :] = (x[src(r), :] * rsqrt(mean(x^2) + eps)) * w   (src/model.zig:1166-1181: scale
// first, weight second).  src(r) = rows ? rows[r] : r.  One block per output row.
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                               TO* __restrict__ y, int dim, float eps) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * dim;
  float ss = 0.f;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    const float v = xr[d];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
  TO* yr = y + (size_t)r * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) yr[d] = from_f32<TO>((xr[d] * scale) * w[d]);
}

// The same with 16-byte loads and the row kept in registers between the sum and the scaling
// (dim a multiple of 4, at most 16 values per thread).  The sum of squares is added per thread
// over its float4s in order, then over the block as above.
template <typename TO>
__global__ void rmsnorm_vec4_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                    const float* __restrict__ w, TO* __restrict__ y, int dim, float eps) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  zk_let_next_start();
  zk_wait_prior();   // x is the kernel before's result
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * dim);
  const int n4 = dim >> 2;
  float4 v[4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    v[i] = d < n4 ? xr[d] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    ss = fmaf(v[i].x, v[i].x, ss);
    ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss);
    ss = fmaf(v[i].w, v[i].w, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
  TO* yr = y + (size_t)r * dim;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    if (d >= n4) continue;
    const float4 wv = reinterpret_cast<const float4*>(w)[d];
    const float o0 = (v[i].x * scale) * wv.x, o1 = (v[i].y * scale) * wv.y, o2 = (v[i].z * scale) * wv.z,
                o3 = (v[i].w * scale) * wv.w;
    if constexpr (sizeof(TO) == 4) {
      reinterpret_cast<float4*>(yr)[d] = make_float4(o0, o1, o2, o3);
    } else {
      __nv_bfloat162 p[2] = {__floats2bfloat162_rn(o0, o1), __floats2bfloat162_rn(o2, o3)};
      reinterpret_cast<uint2*>(yr)[d] = *reinterpret_cast<const uint2*>(p);
    }
  }
}

// h[t, f] = silu(gate_f) * up_f, silu(g) = g / (1 + exp(-g)) (src/ffn.zig:31-33, 49-57).
// A row of gu holds [gate (F) | up (F)] (il = 0), or groups of il gates followed by their il ups
// (il > 0, the layout the fused contraction kernels want).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ h, int n, int F, int il) {
  const size_t total = (size_t)n * F;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / F, f = i - t * F;
    const size_t gi = il ? (f / il) * 2 * il + f % il : f;
    const size_t ui = il ? gi + il : F + f;
    const float g = to_f32(gu[t * 2 * F + gi]);
    const float u = to_f32(gu[t * 2 * F + ui]);
    h[i] = from_f32<T>(g / (1.0f + expf(-g)) * u);
  }
}

// The gated unit of a feed-forward whose gate is capped and whose linear branch is clamped and shifted:
//   g <- min(g, limit), u <- clamp(u, -limit, limit), h = g * sigmoid(alpha * g) * (u + 1)   (float32 arithmetic).
// Rows of gu as in silu_mul_kernel.
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ h, int n, int F, int il, float limit, float alpha) {
  zk_let_next_start();
  zk_wait_prior();
  const size_t total = (size_t)n * F;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / F, f = i - t * F;
    const size_t gi = il ? (f / il) * 2 * il + f % il : f;
    const size_t ui = il ? gi + il : F + f;
    const float g = fminf(to_f32(gu[t * 2 * F + gi]), limit);
    const float u = fminf(fmaxf(to_f32(gu[t * 2 * F + ui]), -limit), limit);
    h[i] = from_f32<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
  }
}

// A gate per (token, head): rows[t, h, :] *= sigmoid(gate[t * ld_gate + h]), gate float32, in place.
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ rows, const float* __restrict__ gate, int ld_gate, int n, int H, int width) {
  zk_let_next_start();
  zk_wait_prior();
  const size_t total = (size_t)n * H * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t th = i / width, t = th / H, hh = th - t * H;
    const float g = gate[t * ld_gate + hh];
    rows[i] = from_f32<T>(to_f32(rows[i]) / (1.0f + expf(-g)));
  }
}

// The same for bfloat16 rows whose heads are whole 16-byte pieces: a thread takes one piece (eight values, one gate).
__global__ void head_gate_vec8_kernel(uint4* __restrict__ rows, const float* __restrict__ gate, int ld_gate, int pieces, int H,
                                      int per_head) {
  zk_let_next_start();
  zk_wait_prior();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pieces) return;
  const int th = i / per_head, t = th / H, hh = th - t * H;
  const float s = 1.0f + expf(-gate[(size_t)t * ld_gate + hh]);
  uint4 v = rows[i];
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(p[j]);
    p[j] = __floats2bfloat162_rn(f.x / s, f.y / s);
  }
  rows[i] = v;
}

// out[i] = mean + std * n_i with n_i standard normal, a function of (seed, i) only: two hashed
// uniforms through Box-Muller.  Fills large random models on the device in milliseconds.
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, size_t n, unsigned long long seed, float mean, float std) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const unsigned long long h = splitmix64(seed ^ splitmix64(i));
    const float u1 = ((float)(unsigned)(h >> 40) + 1.0f) * (1.0f / 16777216.0f);   // (0, 1]
    const float u2 = (float)(unsigned)((h >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);  // [0, 1)
    out[i] = from_f32<T>(mean + std * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2));
  }
}

// x[r, :] += out_scale * ((m[r, :] * rsqrt(mean(m^2) + eps)) * w): the RMSNorm of a sublayer's OUTPUT added to
// the residual rows (out_scale 1), or a share of it (two mixers side by side add half each), all in float32.  One block per row; the row of m stays in registers when it
// fits (16 values per thread), else it is read twice.
__global__ void rmsnorm_add_kernel(const float* __restrict__ m, const float* __restrict__ w, float* __restrict__ x,
                                   int dim, float eps, float out_scale) {
  __shared__ float scratch[32];
  zk_let_next_start();
  zk_wait_prior();
  const int r = blockIdx.x;
  const float* mr = m + (size_t)r * dim;
  float* xr = x + (size_t)r * dim;
  float keep[16];
  const bool fits = dim <= 16 * (int)blockDim.x;
  float ss = 0.f;
  if (fits) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      keep[i] = d < dim ? mr[d] : 0.f;
      ss = fmaf(keep[i], keep[i], ss);
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) ss = fmaf(mr[d], mr[d], ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
  if (fits) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      if (d < dim) xr[d] += out_scale * ((keep[i] * scale) * w[d]);
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) xr[d] += out_scale * ((mr[d] * scale) * w[d]);
  }
}

// The same with 16-byte loads and stores (dim a multiple of 4, at most 16 values per thread, aligned rows).
__global__ void rmsnorm_add_vec4_kernel(const float* __restrict__ m, const float* __restrict__ w, float* __restrict__ x,
                                        int dim, float eps, float out_scale) {
  __shared__ float scratch[32];
  zk_let_next_start();
  zk_wait_prior();
  const int r = blockIdx.x;
  const float4* mr = reinterpret_cast<const float4*>(m + (size_t)r * dim);
  float4* xr = reinterpret_cast<float4*>(x + (size_t)r * dim);
  const int n4 = dim >> 2;
  float4 v[4], xv[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    v[i] = d < n4 ? mr[d] : make_float4(0.f, 0.f, 0.f, 0.f);
    xv[i] = d < n4 ? xr[d] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    ss = fmaf(v[i].x, v[i].x, ss);
    ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss);
    ss = fmaf(v[i].w, v[i].w, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    if (d >= n4) continue;
    const float4 wv = reinterpret_cast<const float4*>(w)[d];
    xr[d] = make_float4(xv[i].x + out_scale * ((v[i].x * scale) * wv.x), xv[i].y + out_scale * ((v[i].y * scale) * wv.y),
                        xv[i].z + out_scale * ((v[i].z * scale) * wv.z), xv[i].w + out_scale * ((v[i].w * scale) * wv.w));
  }
}

// Layer norm: y[r, :] = (x[src(r), :] - mean) / sqrt(var + eps) * w + b, var the mean of the squared deviations
// (two passes over the row, which stays in registers when it fits: 16 values per thread), float32 arithmetic.
// src(r) = rows ? rows[r] : r.  One block per output row; b may be null (no bias).
template <typename TO>
__global__ void layernorm_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                                 const float* __restrict__ b, TO* __restrict__ y, int dim, float eps) {
  __shared__ float scratch[32];
  zk_let_next_start();
  zk_wait_prior();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * dim;
  TO* yr = y + (size_t)r * dim;
  float keep[16];
  const bool fits = dim <= 16 * (int)blockDim.x;
  float sum = 0.f;
  if (fits) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      keep[i] = d < dim ? xr[d] : 0.f;
      sum += keep[i];
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) sum += xr[d];
  }
  const float mean = block_sum(sum, scratch) / (float)dim;
  float ss = 0.f;
  if (fits) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      const float c = d < dim ? keep[i] - mean : 0.f;
      ss = fmaf(c, c, ss);
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      const float c = xr[d] - mean;
      ss = fmaf(c, c, ss);
    }
  }
  const float scale = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dim + eps);
  if (fits) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      if (d < dim) yr[d] = from_f32<TO>(((keep[i] - mean) * scale) * w[d] + (b ? b[d] : 0.f));
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x)
      yr[d] = from_f32<TO>(((xr[d] - mean) * scale) * w[d] + (b ? b[d] : 0.f));
  }
}

// The same with 16-byte loads and the row kept in registers (dim a multiple of 4, at most 16 values per thread, aligned
// rows): one pass over memory.  The sums are added per thread over its float4s in order, then over the block.
template <typename TO>
__global__ void layernorm_vec4_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                                      const float* __restrict__ b, TO* __restrict__ y, int dim, float eps) {
  __shared__ float scratch[32];
  zk_let_next_start();
  zk_wait_prior();
  const int r = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * dim);
  const int n4 = dim >> 2;
  float4 v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    v[i] = d < n4 ? xr[d] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  const float mean = block_sum(sum, scratch) / (float)dim;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if ((int)(threadIdx.x + i * blockDim.x) >= n4) continue;
    v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
    ss = fmaf(v[i].x, v[i].x, ss);
    ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss);
    ss = fmaf(v[i].w, v[i].w, ss);
  }
  const float scale = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dim + eps);
  TO* yr = y + (size_t)r * dim;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    if (d >= n4) continue;
    const float4 wv = reinterpret_cast<const float4*>(w)[d];
    const float4 bv = b ? reinterpret_cast<const float4*>(b)[d] : make_float4(0.f, 0.f, 0.f, 0.f);
    const float o0 = (v[i].x * scale) * wv.x + bv.x, o1 = (v[i].y * scale) * wv.y + bv.y;
    const float o2 = (v[i].z * scale) * wv.z + bv.z, o3 = (v[i].w * scale) * wv.w + bv.w;
    if constexpr (sizeof(TO) == 4) {
      reinterpret_cast<float4*>(yr)[d] = make_float4(o0, o1, o2, o3);
    } else {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
      uint2 packed;
      packed.x = *reinterpret_cast<const unsigned*>(&lo);
      packed.y = *reinterpret_cast<const unsigned*>(&hi);
      reinterpret_cast<uint2*>(yr)[d] = packed;
    }
  }
}

// A gate per value: rows[t, h, j] *= sigmoid(gate[t * ld_gate + h * valid + j]) for j < valid, in place; a head's row is
// `width` values of which the first `valid` are gated (the rest is padding and left alone).  gate float32.
template <typename T>
__global__ void value_gate_kernel(T* __restrict__ rows, const float* __restrict__ gate, int ld_gate, int n, int H, int width,
                                  int valid) {
  zk_let_next_start();
  zk_wait_prior();
  const size_t total = (size_t)n * H * valid;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t th = i / valid, t = th / H;
    const int j = (int)(i - th * valid), hh = (int)(th - t * H);
    const float g = gate[t * ld_gate + (size_t)hh * valid + j];
    T* v = rows + th * width + j;
    *v = from_f32<T>(to_f32(*v) / (1.0f + expf(-g)));
  }
}

// The same for bfloat16 rows in 16-byte pieces (width and valid multiples of 8, gate rows 16-byte aligned).
__global__ void value_gate_vec8_kernel(uint4* __restrict__ rows, const float* __restrict__ gate, int ld_gate, int pieces, int H,
                                       int per_head, int valid_pieces) {
  zk_let_next_start();
  zk_wait_prior();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pieces) return;
  const int th = i / valid_pieces, j = i - th * valid_pieces, t = th / H, hh = th - t * H;
  const float4* g4 = reinterpret_cast<const float4*>(gate + (size_t)t * ld_gate + ((size_t)hh * valid_pieces + j) * 8);
  const float4 ga = g4[0], gb = g4[1];
  const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
  uint4* dst = rows + (size_t)th * per_head + j;
  uint4 v = *dst;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(p[k]);
    p[k] = __floats2bfloat162_rn(f.x / (1.0f + expf(-g[2 * k])), f.y / (1.0f + expf(-g[2 * k + 1])));
  }
  *dst = v;
}

// Heads divided by their root mean square and gated: y[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) *
// silu(gate[t * ld_gate + h * e + :]).  o and gate float32 (o rows packed, H * e wide), y in the run dtype.
// One warp per (token, head); the sum of squares is added in lane order then over the warp's tree.
template <typename TO>
__global__ void unit_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate, int ld_gate,
                                      TO* __restrict__ y, long long items, int H, int e, float eps) {
  zk_let_next_start();
  zk_wait_prior();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  const long long t = item / H;
  const int h = (int)(item - t * H);
  const float* src = o + (size_t)item * e;
  const float* g = gate + (size_t)t * ld_gate + (size_t)h * e;
  float ss = 0.f;
  for (int j = lane; j < e; j += 32) ss = fmaf(src[j], src[j], ss);
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)e + eps);
  for (int j = lane; j < e; j += 32) {
    const float z = g[j];
    y[(size_t)item * e + j] = from_f32<TO>((src[j] * scale) * (z / (1.0f + expf(-z))));
  }
}

// x[r, :] += share * ((a[r, :] * rsqrt(mean(a^2) + eps)) * wa + (b[r, :] * rsqrt(mean(b^2) + eps)) * wb): the results of two
// mixers that ran side by side, each RMS-normalised with a weight of its own, summed into the residual rows in one pass
// (x is read and written once).  Float32; one block per row; both rows stay in registers when they fit (8 values per
// thread each), else they are read twice.
__global__ void rmsnorm_pair_add_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ wa,
                                        const float* __restrict__ wb, float* __restrict__ x, int dim, float eps, float share) {
  __shared__ float scratch[32];
  zk_let_next_start();
  zk_wait_prior();
  const int r = blockIdx.x;
  const float* ar = a + (size_t)r * dim;
  const float* br = b + (size_t)r * dim;
  float* xr = x + (size_t)r * dim;
  float ka[8], kb[8];
  const bool fits = dim <= 8 * (int)blockDim.x;
  float sa = 0.f, sb = 0.f;
  if (fits) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      ka[i] = d < dim ? ar[d] : 0.f;
      kb[i] = d < dim ? br[d] : 0.f;
      sa = fmaf(ka[i], ka[i], sa);
      sb = fmaf(kb[i], kb[i], sb);
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      sa = fmaf(ar[d], ar[d], sa);
      sb = fmaf(br[d], br[d], sb);
    }
  }
  sa = block_sum(sa, scratch);
  sb = block_sum(sb, scratch);
  const float ra = 1.0f / sqrtf(sa / (float)dim + eps), rb = 1.0f / sqrtf(sb / (float)dim + eps);
  if (fits) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      if (d < dim) xr[d] += share * ((ka[i] * ra) * wa[d] + (kb[i] * rb) * wb[d]);
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) xr[d] += share * ((ar[d] * ra) * wa[d] + (br[d] * rb) * wb[d]);
  }
}

// Activations of a plain (ungated) feed-forward, float32 arithmetic:
// 0 = gelu with erf: 0.5 z (1 + erf(z / sqrt 2)); 1 = gelu with tanh:
// 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); 2 = silu; 3 = relu; 4 = the square of relu.
__device__ __forceinline__ float zk_activate(float z, int kind) {
  switch (kind) {
    case 0: return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
    case 1: return 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
    case 2: return z / (1.0f + expf(-z));
    case 4: {
      const float r = fmaxf(z, 0.f);
      return r * r;
    }
    default: return fmaxf(z, 0.f);
  }
}

template <typename T>
__global__ void activation_kernel(const T* __restrict__ in, T* __restrict__ out, size_t total, int kind) {
  zk_let_next_start();
  zk_wait_prior();
  constexpr int PER = 16 / (int)sizeof(T);      // values in 16 bytes
  if (total % PER == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) % 16) == 0) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total / PER; i += (size_t)gridDim.x * blockDim.x) {
      const uint4 raw = reinterpret_cast<const uint4*>(in)[i];
      const T* v = reinterpret_cast<const T*>(&raw);
      uint4 packed;
      T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
      for (int j = 0; j < PER; ++j) o[j] = from_f32<T>(zk_activate(to_f32(v[j]), kind));
      reinterpret_cast<uint4*>(out)[i] = packed;
    }
    return;
  }
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(zk_activate(to_f32(in[i]), kind));
}

// Float32 rows in the run dtype (the input of a contraction that reads the residual rows as they are).
template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ in, T* __restrict__ out, size_t total) {
  zk_let_next_start();
  zk_wait_prior();
  if constexpr (sizeof(T) == 2) {
    if (total % 4 == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) % 16) == 0) {
      for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total / 4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = reinterpret_cast<const float4*>(in)[i];
        __nv_bfloat162 pk[2] = {__floats2bfloat162_rn(v.x, v.y), __floats2bfloat162_rn(v.z, v.w)};
        reinterpret_cast<uint2*>(out)[i] = *reinterpret_cast<const uint2*>(pk);
      }
      return;
    }
  }
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(in[i]);
}

// logits <- cap * tanh(logits / cap), in place, float32.
__global__ void softcap_kernel(float* __restrict__ x, size_t total, float cap) {
  zk_let_next_start();
  zk_wait_prior();
  const float inv = 1.0f / cap;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] * inv);
}

// out = sum_{j < n_terms} w[j] * planes[j], planes [n_terms (or more), plane] float32 one behind the
// other `plane` elements apart, added in the order of j.  n_terms = 1 with w = nullptr copies.
__global__ void weighted_sum_kernel(const float* __restrict__ planes, const float* __restrict__ w, int n_terms,
                                    size_t plane, float* __restrict__ out) {
  zk_let_next_start();
  zk_wait_prior();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < plane; i += (size_t)gridDim.x * blockDim.x) {
    float acc = (w ? w[0] : 1.0f) * planes[i];
    for (int j = 1; j < n_terms; ++j) acc = fmaf(w[j], planes[(size_t)j * plane + i], acc);
    out[i] = acc;
  }
}

// x[t, c] += s[c] * m[t, c]: a sublayer's result m summed into the residual rows through a learned
// scale per channel.  Float32; the product is rounded before the sum (no fused multiply-add), so the
// row is the same whether the scale was applied here or by the kernel that produced m.
__global__ void scale_add_kernel(const float* __restrict__ m, const float* __restrict__ s, float* __restrict__ x,
                                 size_t total, int dim) {
  zk_let_next_start();
  zk_wait_prior();
  if (dim % 4 == 0 && ((reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(x)) % 16) == 0) {
    const int d4 = dim >> 2;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total / 4; i += (size_t)gridDim.x * blockDim.x) {
      const float4 a = reinterpret_cast<const float4*>(m)[i], w = reinterpret_cast<const float4*>(s)[i % d4];
      float4 v = reinterpret_cast<float4*>(x)[i];
      v.x = __fadd_rn(v.x, __fmul_rn(w.x, a.x));
      v.y = __fadd_rn(v.y, __fmul_rn(w.y, a.y));
      v.z = __fadd_rn(v.z, __fmul_rn(w.z, a.z));
      v.w = __fadd_rn(v.w, __fmul_rn(w.w, a.w));
      reinterpret_cast<float4*>(x)[i] = v;
    }
    return;
  }
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    x[i] = __fadd_rn(x[i], __fmul_rn(s[i % dim], m[i]));
}

// x[t, :] = (x[t, :] + base[t, :]) + vec[:]  (base may be absent): what a repeated stretch of layers is
// given before each of its passes, the rows as they left the embedding and a learned vector per pass.
__global__ void rows_add_kernel(float* __restrict__ x, const float* __restrict__ base, const float* __restrict__ vec,
                                size_t total, int dim) {
  zk_let_next_start();
  zk_wait_prior();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float v = x[i];
    if (base) v += base[i];
    x[i] = v + vec[i % dim];
  }
}

// Token shift on normalised rows: n_t = rms(x_t) * w (or x_t itself without w), h_t = n_t + (n_{t-1} - n_t) * mu,
// with n_{t-1} the sequence's previous token's n: the row before in the packed batch, or, for the first
// token a sequence brings in this step, the row `state[slot]` that the step before left (zeros at a
// sequence's start).  One block per token; float32 throughout, h in the run dtype.  n_{t-1} is computed
// again from x_{t-1} with the arithmetic that wrote the state, so a cut between two steps changes no bit.
// With `write_state` (steps of one token per sequence) the block also leaves n_t as the new state;
// otherwise norm_shift_state_kernel does, after every block has read the old one.
__device__ __forceinline__ float row_scale(const float* __restrict__ xr, int dim, float eps, float* scratch) {
  float ss = 0.f;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) ss = fmaf(xr[d], xr[d], ss);
  ss = block_sum(ss, scratch);
  return 1.0f / sqrtf(ss / (float)dim + eps);
}

template <typename TO>
__global__ void norm_shift_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ mu,
                                  float* __restrict__ state, long long state_stride, const int* __restrict__ tok_seq,
                                  const int* __restrict__ cu_q, const int* __restrict__ seq_slot, TO* __restrict__ h,
                                  int dim, float eps, int write_state) {
  __shared__ float scratch[2][32];
  zk_let_next_start();
  zk_wait_prior();
  const int t = blockIdx.x;
  const int b = tok_seq[t];
  const bool first = t == cu_q[b];
  const float* xr = x + (size_t)t * dim;
  const float* xp = first ? nullptr : xr - dim;
  float* st = state + (size_t)seq_slot[b] * state_stride;
  float sc = 1.f, sp = 1.f;
  if (w) {
    sc = row_scale(xr, dim, eps, scratch[0]);
    if (xp) sp = row_scale(xp, dim, eps, scratch[1]);
  }
  TO* hr = h + (size_t)t * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    const float n = w ? (xr[d] * sc) * w[d] : xr[d];
    const float p = xp ? (w ? (xp[d] * sp) * w[d] : xp[d]) : st[d];
    hr[d] = from_f32<TO>(n + (p - n) * mu[d]);
    if (write_state) st[d] = n;
  }
}

// The same for rows of a multiple of four values, at most sixteen per thread: 16-byte loads, and every load of
// the row, the row before, the weights and the state is under way before the first sum is waited for (the plain
// kernel's loads wait for one another; at eight rows of 2,048 values it took 14 us where this form takes 4).
// The sums of squares add a thread's values in the order of the plain kernel's strides only per float4, so the
// two forms may differ in the last bit; a model uses one of them throughout (the choice depends on the width alone).
template <typename TO>
__global__ void norm_shift_vec4_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ mu,
                                       float* __restrict__ state, long long state_stride, const int* __restrict__ tok_seq,
                                       const int* __restrict__ cu_q, const int* __restrict__ seq_slot, TO* __restrict__ h,
                                       int dim, float eps, int write_state) {
  __shared__ float scratch[2][32];
  zk_let_next_start();
  zk_wait_prior();
  const int t = blockIdx.x;
  const int n4 = dim >> 2;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)t * dim);
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f), one = make_float4(1.f, 1.f, 1.f, 1.f);
  float4 vx[4], vp[4], vw[4], vm[4];
  // the row itself, the weights and the shift need no index: they are asked for first
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    const bool in = d < n4;
    vx[i] = in ? xr[d] : zero;
    vw[i] = (in && w) ? reinterpret_cast<const float4*>(w)[d] : one;
    vm[i] = in ? reinterpret_cast<const float4*>(mu)[d] : zero;
  }
  // a sequence's tokens lie side by side in the batch: a token is its sequence's first of this step exactly
  // when the row before belongs to another sequence (two loads that do not wait for one another; the slot,
  // a third one behind them, is needed only by a first token or when the state is written)
  const int b = tok_seq[t];
  const bool first = t == 0 || tok_seq[t - 1] != b;
  const float4* xp = reinterpret_cast<const float4*>(x + (size_t)(first ? t : t - 1) * dim);
  float4* st = (first || write_state) ? reinterpret_cast<float4*>(state + (size_t)seq_slot[b] * state_stride) : nullptr;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    vp[i] = d < n4 ? (first ? st[d] : xp[d]) : zero;
  }
  float sc = 1.f, sp = 1.f;
  if (w) {
    float ss = 0.f, sq = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ss = fmaf(vx[i].x, vx[i].x, ss); ss = fmaf(vx[i].y, vx[i].y, ss); ss = fmaf(vx[i].z, vx[i].z, ss); ss = fmaf(vx[i].w, vx[i].w, ss);
      sq = fmaf(vp[i].x, vp[i].x, sq); sq = fmaf(vp[i].y, vp[i].y, sq); sq = fmaf(vp[i].z, vp[i].z, sq); sq = fmaf(vp[i].w, vp[i].w, sq);
    }
    ss = block_sum(ss, scratch[0]);
    sc = 1.0f / sqrtf(ss / (float)dim + eps);
    if (!first) {
      sq = block_sum(sq, scratch[1]);
      sp = 1.0f / sqrtf(sq / (float)dim + eps);
    }
  }
  const bool norm_prev = w && !first;       // the state already holds a normalised row
  TO* hr = h + (size_t)t * dim;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    if (d >= n4) continue;
    float n[4], p[4], o[4];
    const float xv[4] = {vx[i].x, vx[i].y, vx[i].z, vx[i].w}, pv[4] = {vp[i].x, vp[i].y, vp[i].z, vp[i].w},
                wv[4] = {vw[i].x, vw[i].y, vw[i].z, vw[i].w}, mv[4] = {vm[i].x, vm[i].y, vm[i].z, vm[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      n[j] = w ? (xv[j] * sc) * wv[j] : xv[j];
      p[j] = norm_prev ? (pv[j] * sp) * wv[j] : pv[j];
      o[j] = n[j] + (p[j] - n[j]) * mv[j];
    }
    if constexpr (sizeof(TO) == 4) {
      reinterpret_cast<float4*>(hr)[d] = make_float4(o[0], o[1], o[2], o[3]);
    } else {
      __nv_bfloat162 pk[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
      reinterpret_cast<uint2*>(hr)[d] = *reinterpret_cast<const uint2*>(pk);
    }
    if (write_state) st[d] = make_float4(n[0], n[1], n[2], n[3]);
  }
}

__global__ void norm_shift_state_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ state,
                                        long long state_stride, const int* __restrict__ cu_q,
                                        const int* __restrict__ seq_slot, int dim, float eps, int vec4) {
  // vec4: the sum of squares runs in the order of norm_shift_vec4_kernel (same block size), so that the row left
  // here is bit for bit the row that kernel would compute for a token whose predecessor is in the same step
  __shared__ float scratch[32];
  zk_let_next_start();
  zk_wait_prior();
  const int b = blockIdx.x;
  const int t = cu_q[b + 1] - 1;
  if (t < cu_q[b]) return;
  const float* xr = x + (size_t)t * dim;
  float* st = state + (size_t)seq_slot[b] * state_stride;
  float sc = 1.f;
  if (w && vec4) {
    float ss = 0.f;
    for (int d = threadIdx.x; d < (dim >> 2); d += blockDim.x) {
      const float4 v = reinterpret_cast<const float4*>(xr)[d];
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    ss = block_sum(ss, scratch);
    sc = 1.0f / sqrtf(ss / (float)dim + eps);
  } else if (w) {
    sc = row_scale(xr, dim, eps, scratch);
  }
  for (int d = threadIdx.x; d < dim; d += blockDim.x) st[d] = w ? (xr[d] * sc) * w[d] : xr[d];
}

// m[t, :] += sigmoid(x[t, :] . g) * s[t, :]: a branch s that every token takes, weighed by one
// number per token that a gate vector g [dim] gives.  Float32 throughout; one block per token.
__global__ void gate_add_kernel(const float* __restrict__ x, const float* __restrict__ g, const float* __restrict__ s,
                                float* __restrict__ m, int dim, int out_dim) {
  __shared__ float scratch[32];
  zk_let_next_start();
  zk_wait_prior();
  const int t = blockIdx.x;
  const float* xr = x + (size_t)t * dim;
  const float* sr = s + (size_t)t * out_dim;
  float* mr = m + (size_t)t * out_dim;
  const bool vec = dim % 4 == 0 && out_dim % 4 == 0 &&
                   (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(s) |
                    reinterpret_cast<uintptr_t>(m)) % 16 == 0;
  float dot = 0.f;
  if (vec) {     // the same products, each thread adding its four in order
    for (int d = threadIdx.x; d < dim / 4; d += blockDim.x) {
      const float4 a = reinterpret_cast<const float4*>(xr)[d], b = reinterpret_cast<const float4*>(g)[d];
      dot = fmaf(a.x, b.x, dot);
      dot = fmaf(a.y, b.y, dot);
      dot = fmaf(a.z, b.z, dot);
      dot = fmaf(a.w, b.w, dot);
    }
  } else {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) dot = fmaf(xr[d], g[d], dot);
  }
  dot = block_sum(dot, scratch);
  const float gate = 1.0f / (1.0f + expf(-dot));
  if (vec) {
    for (int d = threadIdx.x; d < out_dim / 4; d += blockDim.x) {
      const float4 a = reinterpret_cast<const float4*>(sr)[d];
      float4 o = reinterpret_cast<float4*>(mr)[d];
      o.x = fmaf(gate, a.x, o.x);
      o.y = fmaf(gate, a.y, o.y);
      o.z = fmaf(gate, a.z, o.z);
      o.w = fmaf(gate, a.w, o.w);
      reinterpret_cast<float4*>(mr)[d] = o;
    }
    return;
  }
  for (int d = threadIdx.x; d < out_dim; d += blockDim.x) mr[d] = fmaf(gate, sr[d], mr[d]);
}

// x *= scale, in place (float32): logits that a design multiplies by a constant.
__global__ void scale_kernel(float* __restrict__ x, size_t total, float scale) {
  zk_let_next_start();
  zk_wait_prior();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) x[i] *= scale;
}

extern "C" {

int zk_fill_normal(void* out, long long n, long long seed, float mean, float std, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
  if (dtype == ZK_F32)
    fill_normal_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, (size_t)n, (unsigned long long)seed, mean, std);
  else if (dtype == ZK_BF16)
    fill_normal_kernel<bf16><<<blocks, threads, 0, stream>>>((bf16*)out, (size_t)n, (unsigned long long)seed, mean, std);
  else
    return ZK_EINVAL;
  return ZK_LAUNCH_STATUS();
}

// Name of a status returned by any zk_* launcher (a cudaError_t value, or ZK_EINVAL).
const char* zk_error_name(int code) {
  if (code == ZK_EINVAL) return "ZK_EINVAL (a size or dtype the kernel does not take)";
  return cudaGetErrorName((cudaError_t)code);
}

int zk_embed(const int* tokens, const void* table, float* x, int n, int dim, int vocab, float scale, int dtype,
             int* status, const void* pos_table, const int* tok_pos, int max_pos, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dim <= 0 || vocab <= 0 || (pos_table && (!tok_pos || max_pos <= 0))) return ZK_EINVAL;
  const int threads = dim >= 1024 ? 256 : 128;
  if (dtype == ZK_F32)
    embed_kernel<float><<<n, threads, 0, stream>>>(tokens, (const float*)table, x, dim, vocab, scale, status,
                                                   (const float*)pos_table, tok_pos, max_pos);
  else if (dtype == ZK_BF16)
    embed_kernel<bf16><<<n, threads, 0, stream>>>(tokens, (const bf16*)table, x, dim, vocab, scale, status,
                                                  (const bf16*)pos_table, tok_pos, max_pos);
  else
    return ZK_EINVAL;
  return ZK_LAUNCH_STATUS();
}

int zk_rmsnorm(const float* x, const int* rows, const float* w, void* y, int n_out, int dim, float eps, int out_dtype,
               cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (dim <= 0) return ZK_EINVAL;
  int threads = 32;
  while (threads < 256 && threads * 4 < dim) threads <<= 1;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) % 16 == 0;
  if (dim % 4 == 0 && dim <= 16 * threads && aligned && (out_dtype == ZK_F32 || out_dtype == ZK_BF16)) {
    while (threads > 32 && threads * 4 >= 2 * dim) threads >>= 1;   // no idle warps for short rows
    if (out_dtype == ZK_F32)
      return zk_launch_dependent(rmsnorm_vec4_kernel<float>, dim3(n_out), dim3(threads), 0, stream, x, rows, w, (float*)y, dim, eps);
    return zk_launch_dependent(rmsnorm_vec4_kernel<bf16>, dim3(n_out), dim3(threads), 0, stream, x, rows, w, (bf16*)y, dim, eps);
  }
  if (out_dtype == ZK_F32)
    rmsnorm_kernel<float><<<n_out, threads, 0, stream>>>(x, rows, w, (float*)y, dim, eps);
  else if (out_dtype == ZK_BF16)
    rmsnorm_kernel<bf16><<<n_out, threads, 0, stream>>>(x, rows, w, (bf16*)y, dim, eps);
  else
    return ZK_EINVAL;
  return ZK_LAUNCH_STATUS();
}

int zk_silu_mul(const void* gu, void* h, int n, int F, int il, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (F <= 0 || il < 0 || (il > 0 && F % il)) return ZK_EINVAL;
  const size_t total = (size_t)n * F;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == ZK_F32)
    silu_mul_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)h, n, F, il);
  else if (dtype == ZK_BF16)
    silu_mul_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)h, n, F, il);
  else
    return ZK_EINVAL;
  return ZK_LAUNCH_STATUS();
}

static inline int grid_for_total(size_t total, int threads) {
  const size_t want = (total + threads - 1) / threads;
  return (int)(want < 148 * 16 ? want : 148 * 16);
}

int zk_rmsnorm_add(const float* m, const float* w, float* x, int n, int dim, float eps, float out_scale,
                   cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dim <= 0) return ZK_EINVAL;
  int threads = 32;
  while (threads < 256 && threads * 4 < dim) threads <<= 1;
  const bool aligned = (reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) % 16 == 0;
  if (dim % 4 == 0 && dim <= 16 * threads && aligned) {
    while (threads > 32 && threads * 4 >= 2 * dim) threads >>= 1;   // no idle warps for short rows
    return zk_launch_dependent(rmsnorm_add_vec4_kernel, dim3(n), dim3(threads), 0, stream, m, w, x, dim, eps, out_scale);
  }
  return zk_launch_dependent(rmsnorm_add_kernel, dim3(n), dim3(threads), 0, stream, m, w, x, dim, eps, out_scale);
}

int zk_rmsnorm_pair_add(const float* a, const float* b, const float* wa, const float* wb, float* x, int n, int dim, float eps,
                        float share, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dim <= 0) return ZK_EINVAL;
  int threads = 32;
  while (threads < 256 && threads * 8 < dim) threads <<= 1;
  return zk_launch_dependent(rmsnorm_pair_add_kernel, dim3(n), dim3(threads), 0, stream, a, b, wa, wb, x, dim, eps, share);
}

int zk_activation(const void* in, void* out, long long total, int kind, int dtype, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (kind < 0 || kind > 4) return ZK_EINVAL;
  const int threads = 256, blocks = grid_for_total((size_t)total, threads);
  if (dtype == ZK_F32)
    return zk_launch_dependent(activation_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)in, (float*)out, (size_t)total, kind);
  if (dtype == ZK_BF16)
    return zk_launch_dependent(activation_kernel<bf16>, dim3(blocks), dim3(threads), 0, stream, (const bf16*)in, (bf16*)out, (size_t)total, kind);
  return ZK_EINVAL;
}

int zk_cast_rows(const float* in, void* out, long long total, int dtype, cudaStream_t stream) {
  if (total <= 0) return 0;
  const int threads = 256, blocks = grid_for_total((size_t)total, threads);
  if (dtype == ZK_F32)
    return zk_launch_dependent(cast_rows_kernel<float>, dim3(blocks), dim3(threads), 0, stream, in, (float*)out, (size_t)total);
  if (dtype == ZK_BF16)
    return zk_launch_dependent(cast_rows_kernel<bf16>, dim3(blocks), dim3(threads), 0, stream, in, (bf16*)out, (size_t)total);
  return ZK_EINVAL;
}

int zk_softcap(float* x, long long total, float cap, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (!(cap > 0.f)) return ZK_EINVAL;
  const int threads = 256, blocks = grid_for_total((size_t)total, threads);
  return zk_launch_dependent(softcap_kernel, dim3(blocks), dim3(threads), 0, stream, x, (size_t)total, cap);
}

int zk_scale(float* x, long long total, float scale, cudaStream_t stream) {
  if (total <= 0) return 0;
  const int threads = 256, blocks = grid_for_total((size_t)total, threads);
  return zk_launch_dependent(scale_kernel, dim3(blocks), dim3(threads), 0, stream, x, (size_t)total, scale);
}

int zk_weighted_sum(const float* planes, const float* w, int n_terms, long long plane, float* out, cudaStream_t stream) {
  if (plane <= 0) return 0;
  if (n_terms < 1 || (n_terms > 1 && !w)) return ZK_EINVAL;
  const int threads = 256, blocks = grid_for_total((size_t)plane, threads);
  return zk_launch_dependent(weighted_sum_kernel, dim3(blocks), dim3(threads), 0, stream, planes, w, n_terms, (size_t)plane, out);
}

int zk_scale_add(const float* m, const float* s, float* x, long long total, int dim, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (dim <= 0 || total % dim) return ZK_EINVAL;
  const int threads = 256, blocks = grid_for_total((size_t)total / (dim % 4 == 0 ? 4 : 1), threads);
  return zk_launch_dependent(scale_add_kernel, dim3(blocks), dim3(threads), 0, stream, m, s, x, (size_t)total, dim);
}

int zk_rows_add(float* x, const float* base, const float* vec, long long total, int dim, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (dim <= 0 || total % dim || !vec) return ZK_EINVAL;
  const int threads = 256, blocks = grid_for_total((size_t)total, threads);
  return zk_launch_dependent(rows_add_kernel, dim3(blocks), dim3(threads), 0, stream, x, base, vec, (size_t)total, dim);
}

// Token shift (see norm_shift_kernel).  x float32 [n, dim]; w [dim] or null; mu [dim]; state rows
// `state_stride` floats apart, one per slot; h [n, dim] in out_dtype.
int zk_norm_shift(const float* x, const float* w, const float* mu, float* state, long long state_stride,
                  const int* tok_seq, const int* cu_q, const int* seq_slot, void* h, int n, int n_seqs, int dim, float eps,
                  int single_token, int out_dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dim <= 0 || n_seqs <= 0 || !mu || !state) return ZK_EINVAL;
  int threads = 32;
  while (threads < 256 && threads * 4 < dim) threads <<= 1;
  if (out_dtype != ZK_F32 && out_dtype != ZK_BF16) return ZK_EINVAL;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(mu) |
                        reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(h)) % 16 == 0 && state_stride % 4 == 0;
  const bool vec4 = dim % 4 == 0 && dim <= 16 * threads && aligned;
  int rc;
  if (vec4) {
    while (threads > 32 && threads * 4 >= 2 * dim) threads >>= 1;   // no idle warps for short rows
    rc = out_dtype == ZK_F32
             ? zk_launch_dependent(norm_shift_vec4_kernel<float>, dim3(n), dim3(threads), 0, stream, x, w, mu, state,
                                   state_stride, tok_seq, cu_q, seq_slot, (float*)h, dim, eps, single_token ? 1 : 0)
             : zk_launch_dependent(norm_shift_vec4_kernel<bf16>, dim3(n), dim3(threads), 0, stream, x, w, mu, state,
                                   state_stride, tok_seq, cu_q, seq_slot, (bf16*)h, dim, eps, single_token ? 1 : 0);
  } else {
    rc = out_dtype == ZK_F32
             ? zk_launch_dependent(norm_shift_kernel<float>, dim3(n), dim3(threads), 0, stream, x, w, mu, state, state_stride,
                                   tok_seq, cu_q, seq_slot, (float*)h, dim, eps, single_token ? 1 : 0)
             : zk_launch_dependent(norm_shift_kernel<bf16>, dim3(n), dim3(threads), 0, stream, x, w, mu, state, state_stride,
                                   tok_seq, cu_q, seq_slot, (bf16*)h, dim, eps, single_token ? 1 : 0);
  }
  if (rc != 0 || single_token) return rc;
  return zk_launch_dependent(norm_shift_state_kernel, dim3(n_seqs), dim3(threads), 0, stream, x, w, state, state_stride,
                             cu_q, seq_slot, dim, eps, vec4 ? 1 : 0);
}

int zk_clamped_glu(const void* gu, void* h, int n, int F, int il, float limit, float alpha, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (F <= 0 || il < 0 || (il > 0 && F % il)) return ZK_EINVAL;
  const int threads = 256, blocks = grid_for_total((size_t)n * F, threads);
  if (dtype == ZK_F32)
    return zk_launch_dependent(clamped_glu_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)gu, (float*)h, n, F, il, limit, alpha);
  if (dtype == ZK_BF16)
    return zk_launch_dependent(clamped_glu_kernel<bf16>, dim3(blocks), dim3(threads), 0, stream, (const bf16*)gu, (bf16*)h, n, F, il, limit, alpha);
  return ZK_EINVAL;
}

int zk_head_gate(void* rows, const float* gate, int ld_gate, int n, int H, int width, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (H <= 0 || width <= 0 || ld_gate < H) return ZK_EINVAL;
  if (dtype == ZK_BF16 && width % 8 == 0 && (uintptr_t)rows % 16 == 0 && (size_t)n * H * (width / 8) < 0x7fffffffULL) {
    const int pieces = n * H * (width / 8);
    return zk_launch_dependent(head_gate_vec8_kernel, dim3((pieces + 255) / 256), dim3(256), 0, stream, (uint4*)rows, gate,
                               ld_gate, pieces, H, width / 8);
  }
  const int threads = 256, blocks = grid_for_total((size_t)n * H * width, threads);
  if (dtype == ZK_F32)
    return zk_launch_dependent(head_gate_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (float*)rows, gate, ld_gate, n, H, width);
  if (dtype == ZK_BF16)
    return zk_launch_dependent(head_gate_kernel<bf16>, dim3(blocks), dim3(threads), 0, stream, (bf16*)rows, gate, ld_gate, n, H, width);
  return ZK_EINVAL;
}

// Layer norm of float32 rows (all, or those listed in `rows`) with weight and optional bias into `out_dtype`.
int zk_layernorm(const float* x, const int* rows, const float* w, const float* b, void* y, int n_out, int dim, float eps,
                 int out_dtype, cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (dim <= 0 || !w) return ZK_EINVAL;
  int threads = 32;
  while (threads < 256 && threads * 4 < dim) threads <<= 1;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(b) |
                        reinterpret_cast<uintptr_t>(y)) % 16 == 0;
  if (dim % 4 == 0 && dim <= 16 * threads && aligned && (out_dtype == ZK_F32 || out_dtype == ZK_BF16)) {
    while (threads > 32 && threads * 4 >= 2 * dim) threads >>= 1;   // no idle warps for short rows
    if (out_dtype == ZK_F32)
      return zk_launch_dependent(layernorm_vec4_kernel<float>, dim3(n_out), dim3(threads), 0, stream, x, rows, w, b, (float*)y, dim, eps);
    return zk_launch_dependent(layernorm_vec4_kernel<bf16>, dim3(n_out), dim3(threads), 0, stream, x, rows, w, b, (bf16*)y, dim, eps);
  }
  if (out_dtype == ZK_F32)
    return zk_launch_dependent(layernorm_kernel<float>, dim3(n_out), dim3(threads), 0, stream, x, rows, w, b, (float*)y, dim, eps);
  if (out_dtype == ZK_BF16)
    return zk_launch_dependent(layernorm_kernel<bf16>, dim3(n_out), dim3(threads), 0, stream, x, rows, w, b, (bf16*)y, dim, eps);
  return ZK_EINVAL;
}

// rows [n, H * width] (run dtype) gated value by value: gate float32, rows `ld_gate` apart, H * valid logits a row.
int zk_value_gate(void* rows, const float* gate, int ld_gate, int n, int H, int width, int valid, int dtype,
                  cudaStream_t stream) {
  if (n <= 0) return 0;
  if (H <= 0 || width <= 0 || valid <= 0 || valid > width || ld_gate < H * valid) return ZK_EINVAL;
  if (dtype == ZK_BF16 && width % 8 == 0 && valid % 8 == 0 && ld_gate % 4 == 0 && (uintptr_t)rows % 16 == 0 &&
      (uintptr_t)gate % 16 == 0 && (size_t)n * H * (valid / 8) < 0x7fffffffULL) {
    const int pieces = n * H * (valid / 8);
    return zk_launch_dependent(value_gate_vec8_kernel, dim3((pieces + 255) / 256), dim3(256), 0, stream, (uint4*)rows, gate,
                               ld_gate, pieces, H, width / 8, valid / 8);
  }
  const int threads = 256, blocks = grid_for_total((size_t)n * H * valid, threads);
  if (dtype == ZK_F32)
    return zk_launch_dependent(value_gate_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (float*)rows, gate, ld_gate, n, H, width, valid);
  if (dtype == ZK_BF16)
    return zk_launch_dependent(value_gate_kernel<bf16>, dim3(blocks), dim3(threads), 0, stream, (bf16*)rows, gate, ld_gate, n, H, width, valid);
  return ZK_EINVAL;
}

// y [n, H * e] (out_dtype) = every head of o [n, H * e] (float32) over its root mean square, times silu(gate).
int zk_unit_norm_gate(const float* o, const float* gate, int ld_gate, void* y, int n, int H, int e, float eps, int out_dtype,
                      cudaStream_t stream) {
  if (n <= 0) return 0;
  if (H <= 0 || e <= 0 || ld_gate < H * e) return ZK_EINVAL;
  const long long items = (long long)n * H;
  const int warps = 4;
  const int blocks = (int)((items + warps - 1) / warps);
  if (out_dtype == ZK_F32)
    return zk_launch_dependent(unit_norm_gate_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, o, gate, ld_gate, (float*)y, items, H, e, eps);
  if (out_dtype == ZK_BF16)
    return zk_launch_dependent(unit_norm_gate_kernel<bf16>, dim3(blocks), dim3(warps * 32), 0, stream, o, gate, ld_gate, (bf16*)y, items, H, e, eps);
  return ZK_EINVAL;
}

int zk_gate_add(const float* x, const float* g, const float* s, float* m, int n, int dim, int out_dim, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dim <= 0 || out_dim <= 0) return ZK_EINVAL;
  int threads = 32;
  while (threads < 256 && threads * 4 < dim) threads <<= 1;
  return zk_launch_dependent(gate_add_kernel, dim3(n), dim3(threads), 0, stream, x, g, s, m, dim, out_dim);
}

}  // extern "C"
