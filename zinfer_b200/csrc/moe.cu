// Mixture of small gated feed-forwards whose experts are picked by a TABLE indexed with the token id
// (no router): token t uses experts table[token_t][0 .. top), each with weight 1/top.
//   y_t = (1/top) * sum_k W_down[e_k] (silu(W_gate[e_k] x_t) * (W_up[e_k] x_t))
// Two weight-streaming kernels.  (1) gate/up: one block per (token, k) and slice of the expert's
// hidden units; a warp owns a hidden unit at a time, its lanes walk the input row, sums in float32,
// silu in float32.  (2) down: one block per token and slice of the outputs; the `top` experts are
// added in the order of k, so a token's result does not depend on the rest of the batch.
// Weights are stacked in the run dtype: gate and up as ONE tensor [experts, 2F, D] whose rows are
// [gate (F) | up (F)] (il = 0) or groups of il gate rows followed by their il up rows (il > 0, the layout
// the contraction kernels with an activation epilogue want), down as [experts, D, F]; x and h are the run
// dtype, y float32.
//
// For steps of many tokens there are two helper kernels instead: rows gathered in the order of their
// experts (so that each expert's rows are one contiguous matrix for a tensor-core contraction) and the
// weighted sum of a token's `top` result rows, added in the order of k.
#include "common.cuh"
#include <stdint.h>

#define MOE_WARPS 8

template <typename T> struct Vec8;   // eight consecutive values as float
template <> struct Vec8<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float* o) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      o[2 * i] = f.x;
      o[2 * i + 1] = f.y;
    }
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float* o) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
  }
};

// R dot products at once: weight rows w[0..R) with the row staged in shared memory (float32), lanes
// striding.  All R loads of a step are requested before the first is used, so a warp keeps R x 512 bytes
// in flight; one row at a time the kernel waited for memory once per row.  VEC: rows are 16-byte aligned
// and K a multiple of 8.  Each sum is added in the same order whatever R is and whichever rows share the call.
template <typename T, bool VEC, int R>
__device__ __forceinline__ void rows_dot(const T* const (&w)[R], const float* __restrict__ xs, int K, int lane,
                                         float (&out)[R]) {
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  if (VEC) {
    for (int k = lane * 8; k < K; k += 256) {
      float v[R][8];
#pragma unroll
      for (int r = 0; r < R; ++r) Vec8<T>::load(w[r] + k, v[r]);
      float x[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = xs[k + i];
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r] = fmaf(v[r][i], x[i], acc[r]);
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      const float x = xs[k];
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = fmaf(to_f32(w[r][k]), x, acc[r]);
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) out[r] = warp_sum(acc[r]);
}

#define MOE_UNITS 4      // hidden units (gate and up row each) or outputs a warp works on at once

// With `tokens` null the experts are not looked up through a table: `table` is then [n, top], the experts a
// router chose for each token.
// Ids n_experts .. n_experts + n_ident - 1 name identity experts (no weights: the expert's output is its input).
__device__ __forceinline__ int moe_expert(const int* __restrict__ tokens, const int* __restrict__ table, int t, int k,
                                          int top, int vocab, int n_experts, int* status, int n_ident = 0) {
  if (!tokens) {
    int e = table[(size_t)t * top + k];
    if (e < 0 || e >= n_experts + n_ident) {
      if (threadIdx.x == 0) atomicExch(status, 4);
      e = 0;
    }
    return e;
  }
  int tok = tokens[t];
  if (tok < 0 || tok >= vocab) tok = 0;        // the embedding kernel has flagged it
  int e = table[(size_t)tok * top + k];
  if (e < 0 || e >= n_experts) {
    if (threadIdx.x == 0) atomicExch(status, 4);
    e = 0;
  }
  return e;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(MOE_WARPS * 32)
    moe_gate_up_kernel(const T* __restrict__ x, const int* __restrict__ tokens, const int* __restrict__ table,
                       const T* __restrict__ w_gu, int il, T* __restrict__ h, int D, int F,
                       int top, int vocab, int n_experts, int units_per_block, int* status, int n_ident) {
  extern __shared__ float xs[];     // [D]
  zk_let_next_start();
  zk_wait_prior();
  const int t = blockIdx.x / top, k = blockIdx.x % top;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e = moe_expert(tokens, table, t, k, top, vocab, n_experts, status, n_ident);
  if (e >= n_experts) return;       // an identity expert has no hidden units
  for (int d = threadIdx.x; d < D; d += blockDim.x) xs[d] = to_f32(x[(size_t)t * D + d]);
  __syncthreads();
  const T* w = w_gu + (size_t)e * 2 * F * D;
  const int f0 = blockIdx.y * units_per_block, f1 = min(F, f0 + units_per_block);
  for (int fb = f0 + warp * MOE_UNITS; fb < f1; fb += MOE_WARPS * MOE_UNITS) {
    const T* rows[2 * MOE_UNITS];
#pragma unroll
    for (int u = 0; u < MOE_UNITS; ++u) {
      const int f = min(fb + u, f1 - 1);        // a unit beyond the slice repeats the last one and is not written
      const int grow = il ? (f / il) * 2 * il + f % il : f;
      const int urow = il ? grow + il : F + f;
      rows[2 * u] = w + (size_t)grow * D;
      rows[2 * u + 1] = w + (size_t)urow * D;
    }
    float dot[2 * MOE_UNITS];
    rows_dot<T, VEC, 2 * MOE_UNITS>(rows, xs, D, lane, dot);
    if (lane < MOE_UNITS && fb + lane < f1) {
      float g = 0.f, u = 0.f;
#pragma unroll
      for (int i = 0; i < MOE_UNITS; ++i)
        if (lane == i) {
          g = dot[2 * i];
          u = dot[2 * i + 1];
        }
      h[((size_t)t * top + k) * F + fb + lane] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(MOE_WARPS * 32)
    moe_down_kernel(const T* __restrict__ h, const int* __restrict__ tokens, const int* __restrict__ table,
                    const T* __restrict__ w_down, float* __restrict__ y, int D, int F, int top, int vocab,
                    int n_experts, int outs_per_block, int accumulate, int* status, const float* __restrict__ route_w,
                    int n_ident, const T* __restrict__ x) {
  // route_w [n, top]: the weight of each of the token's experts (null: 1/top each).  x [n, D]: the rows the experts
  // read, which an identity expert (n_ident > 0) hands on as they are.
  extern __shared__ float hs[];     // [top][F]
  zk_let_next_start();
  zk_wait_prior();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < top * F; i += blockDim.x) hs[i] = to_f32(h[(size_t)t * top * F + i]);
  __syncthreads();
  const float weight = 1.0f / (float)top;
  const int d0 = blockIdx.y * outs_per_block, d1 = min(D, d0 + outs_per_block);
  for (int db = d0 + warp * MOE_UNITS; db < d1; db += MOE_WARPS * MOE_UNITS) {
    float acc[MOE_UNITS];
#pragma unroll
    for (int u = 0; u < MOE_UNITS; ++u) acc[u] = 0.f;
    for (int k = 0; k < top; ++k) {
      const int e = moe_expert(tokens, table, t, k, top, vocab, n_experts, status, n_ident);
      if (e >= n_experts) {          // identity: the weight times the input row
        const float wi = route_w ? route_w[(size_t)t * top + k] : weight;
#pragma unroll
        for (int u = 0; u < MOE_UNITS; ++u) acc[u] += wi * to_f32(x[(size_t)t * D + min(db + u, d1 - 1)]);
        continue;
      }
      const T* rows[MOE_UNITS];
#pragma unroll
      for (int u = 0; u < MOE_UNITS; ++u) rows[u] = w_down + ((size_t)e * D + min(db + u, d1 - 1)) * F;
      float dot[MOE_UNITS];
      rows_dot<T, VEC, MOE_UNITS>(rows, hs + (size_t)k * F, F, lane, dot);
#pragma unroll
      const float wk = route_w ? route_w[(size_t)t * top + k] : weight;
#pragma unroll
      for (int u = 0; u < MOE_UNITS; ++u) acc[u] += wk * dot[u];
    }
    if (lane < MOE_UNITS && db + lane < d1) {
      float v = 0.f;
#pragma unroll
      for (int u = 0; u < MOE_UNITS; ++u)
        if (lane == u) v = acc[u];
      float* dst = y + (size_t)t * D + db + lane;
      *dst = accumulate ? *dst + v : v;
    }
  }
}

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ row_token, T* __restrict__ xg, int D) {
  zk_let_next_start();
  zk_wait_prior();
  const int t = row_token[blockIdx.x];       // < 0: a padding row
  const T* src = x + (size_t)(t < 0 ? 0 : t) * D;
  T* dst = xg + (size_t)blockIdx.x * D;
  constexpr int PER = 16 / (int)sizeof(T);
  if (D % PER == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(xg)) % 16) == 0) {   // rows in 16-byte pieces
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int d = threadIdx.x; d < D / PER; d += blockDim.x)
      reinterpret_cast<uint4*>(dst)[d] = t < 0 ? zero : reinterpret_cast<const uint4*>(src)[d];
    return;
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) dst[d] = t < 0 ? from_f32<T>(0.f) : src[d];
}

// The rows of a prompt step sorted by expert, made where the router left its choice (no trip to the host):
// ids [P] names the expert of pair i = t * top + k.  Expert e's pairs get the rows start_e .. start_e + count_e - 1,
// start_e a multiple of `tile` (every expert's rows are padded to whole tiles); row_token [cap] = the token of each
// row, -1 for a padding row; pair_row [P] = the row of each pair; tile_group [cap / tile] = the expert of each tile
// (0 for the tiles behind the last expert's, whose rows are all padding).  cap >= P rounded down to tiles plus one
// tile per expert.  One block; the order of an expert's rows is not fixed, which no row's result depends on.
__global__ void __launch_bounds__(1024)
    moe_expert_rows_kernel(const int* __restrict__ ids, int P, int E, int top, int tile, int cap,
                           int* __restrict__ row_token, int* __restrict__ pair_row, int* __restrict__ tile_group, int n_ident) {
  extern __shared__ int sh[];      // count [E], start [E]
  int* count = sh;
  int* start = sh + E;
  zk_let_next_start();
  zk_wait_prior();
  const int tid = threadIdx.x, nt = blockDim.x;
  for (int e = tid; e < E; e += nt) count[e] = 0;
  for (int i = tid; i < cap; i += nt) row_token[i] = -1;
  __syncthreads();
  // a pair whose id names an identity expert (E .. E + n_ident - 1) gets no row: pair_row = -1
  for (int i = tid; i < P; i += nt)
    if (!(n_ident > 0 && ids[i] >= E)) atomicAdd(&count[min(max(ids[i], 0), E - 1)], 1);
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = run;
      const int tiles = (count[e] + tile - 1) / tile;
      for (int t = 0; t < tiles; ++t) tile_group[run / tile + t] = e;
      run += tiles * tile;
      count[e] = 0;            // from here on the expert's next free row
    }
    for (int t = run / tile; t < cap / tile; ++t) tile_group[t] = 0;
  }
  __syncthreads();
  for (int i = tid; i < P; i += nt) {
    if (n_ident > 0 && ids[i] >= E) {
      pair_row[i] = -1;
      continue;
    }
    const int e = min(max(ids[i], 0), E - 1);
    const int r = start[e] + atomicAdd(&count[e], 1);
    row_token[r] = i / top;
    pair_row[i] = r;
  }
}

// A pair without a row (pair_row < 0) stands for an identity expert: its term is the weight times the token's own input
// row x[t] (run dtype: float32 or, with x_bf16, bfloat16).
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pair_row, float* __restrict__ out,
                                   int D, int top, int accumulate, const float* __restrict__ route_w,
                                   const void* __restrict__ x, int x_bf16) {
  zk_let_next_start();
  zk_wait_prior();
  const int t = blockIdx.x;
  const float weight = 1.0f / (float)top;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int r = pair_row[t * top + k];
      float term;
      if (r >= 0) term = y[(size_t)r * D + d];
      else if (!x) term = 0.f;
      else term = x_bf16 ? to_f32(reinterpret_cast<const bf16*>(x)[(size_t)t * D + d]) : reinterpret_cast<const float*>(x)[(size_t)t * D + d];
      acc += (route_w ? route_w[(size_t)t * top + k] : weight) * term;
    }
    out[(size_t)t * D + d] = accumulate ? out[(size_t)t * D + d] + acc : acc;
  }
}

// Router of a mixture of experts, one block per token.  The logits are float32 dot products (a warp per expert,
// lanes striding the row, sums in lane order then the warp's tree), the softmax runs over all E experts, and warp 0
// then picks the `top` largest scores one after the other (of equal scores the lower index first).
#define MOE_ROUTER_MAX_EXPERTS 4096
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
    moe_router_kernel(const T* __restrict__ x, const float* __restrict__ w, int* __restrict__ ids, float* __restrict__ wts,
                      int D, int E, int top, const float* __restrict__ correction) {
  // correction [E] (or null): the experts are CHOSEN by score + correction; the weights use the scores alone.
  extern __shared__ float rs[];     // [D] the token's row, [E] logits then scores, [E] what the choice looks at
  float* xs = rs;
  float* z = rs + D;
  float* pick = z + E;
  zk_let_next_start();
  zk_wait_prior();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int d = threadIdx.x; d < D; d += blockDim.x) xs[d] = to_f32(x[(size_t)t * D + d]);
  __syncthreads();
  for (int e = warp; e < E; e += MOE_WARPS) {
    const float* wr = w + (size_t)e * D;
    float acc = 0.f;
    if ((D & 3) == 0) {          // rows in pieces of four: a quarter of the loads (D is the model's: one order per model)
      const float4* w4 = reinterpret_cast<const float4*>(wr);
      const float4* x4 = reinterpret_cast<const float4*>(xs);
      for (int d = lane; d < (D >> 2); d += 32) {
        const float4 a = w4[d], v = x4[d];
        acc = fmaf(a.x, v.x, acc);
        acc = fmaf(a.y, v.y, acc);
        acc = fmaf(a.z, v.z, acc);
        acc = fmaf(a.w, v.w, acc);
      }
    } else {
      for (int d = lane; d < D; d += 32) acc = fmaf(wr[d], xs[d], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) z[e] = acc;
  }
  __syncthreads();
  if (warp != 0) return;
  float m = -INFINITY;
  for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
  m = warp_max(m);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float v = expf(z[e] - m);
    z[e] = v;
    sum += v;
  }
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < E; e += 32) pick[e] = correction ? z[e] / sum + correction[e] : z[e];
  __syncwarp();
  float chosen_sum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int arg = E;
    for (int e = lane; e < E; e += 32)
      if (pick[e] > best) {       // ascending e within a lane: the lower index wins a tie
        best = pick[e];
        arg = e;
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) {
        best = ob;
        arg = oa;
      }
    }
    arg = min(arg, E - 1);        // (only scores that are no numbers leave arg at E)
    const float score = z[arg] / sum;
    __syncwarp();
    if (lane == 0) {
      ids[(size_t)t * top + k] = arg;
      wts[(size_t)t * top + k] = score;
      pick[arg] = -INFINITY;      // taken
    }
    chosen_sum += score;
    __syncwarp();
  }
  const float inv = 1.0f / (chosen_sum + 1e-20f);
  __syncwarp();
  for (int k = lane; k < top; k += 32) wts[(size_t)t * top + k] *= inv;
}

namespace {

template <typename T>
int launch_moe(const void* x, const int* tokens, const int* table, const void* w_gu, int il,
               const void* w_down, void* h, float* y, int n, int D, int F, int top, int vocab, int n_experts,
               int accumulate, int* status, const float* route_w, int n_ident, cudaStream_t stream) {
  const int per = 16 / (int)sizeof(T);   // elements per 16 bytes
  auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec_gu = D % 8 == 0 && D % per == 0 && aligned(w_gu);
  const bool vec_dn = F % 8 == 0 && F % per == 0 && aligned(w_down);
  // enough blocks to fill the GPU when the tokens are few, whole experts per block when they are many
  int units = F, outs = D;
  const long long pairs = (long long)n * top;
  constexpr int GRAIN = MOE_WARPS * MOE_UNITS;     // what a block's warps take in one round
  while (units > GRAIN && pairs * ((F + units - 1) / units) < 2 * 148) units = (units + 1) / 2;
  while (outs > GRAIN && (long long)n * ((D + outs - 1) / outs) < 2 * 148) outs = (outs + 1) / 2;
  units = (units + GRAIN - 1) / GRAIN * GRAIN;
  outs = (outs + GRAIN - 1) / GRAIN * GRAIN;
  const size_t smem_gu = sizeof(float) * D, smem_dn = sizeof(float) * (size_t)top * F;
  if (smem_gu > 200 * 1024 || smem_dn > 200 * 1024) return ZK_EINVAL;
  const dim3 grid_gu((unsigned)pairs, (F + units - 1) / units), grid_dn(n, (D + outs - 1) / outs);
  int rc;
#define ZK_MOE_GU(V)                                                                                                  \
  do {                                                                                                                \
    auto kern = moe_gate_up_kernel<T, V>;                                                                             \
    if (smem_gu > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_gu);          \
      if (e != cudaSuccess) return (int)e;                                                                            \
    }                                                                                                                 \
    rc = zk_launch_dependent(kern, grid_gu, dim3(MOE_WARPS * 32), smem_gu, stream, (const T*)x, tokens, table,        \
                             (const T*)w_gu, il, (T*)h, D, F, top, vocab, n_experts, units, status, n_ident);         \
  } while (0)
#define ZK_MOE_DN(V)                                                                                                  \
  do {                                                                                                                \
    auto kern = moe_down_kernel<T, V>;                                                                                \
    if (smem_dn > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dn);          \
      if (e != cudaSuccess) return (int)e;                                                                            \
    }                                                                                                                 \
    rc = zk_launch_dependent(kern, grid_dn, dim3(MOE_WARPS * 32), smem_dn, stream, (const T*)h, tokens, table,        \
                             (const T*)w_down, y, D, F, top, vocab, n_experts, outs, accumulate, status, route_w,     \
                             n_ident, (const T*)x);                                                                   \
  } while (0)
  if (vec_gu) ZK_MOE_GU(true); else ZK_MOE_GU(false);
  if (rc != 0) return rc;
  if (vec_dn) ZK_MOE_DN(true); else ZK_MOE_DN(false);
  return rc;
#undef ZK_MOE_GU
#undef ZK_MOE_DN
}

}  // namespace

extern "C" {

// x [n, D], h [n, top, F] (scratch, run dtype), y [n, D] float32 (= or += with `accumulate`);
// tokens [n] and table [vocab, top] int32; w_gu [experts, 2F, D] (see `il` above), w_down [experts, D, F].
int zk_moe_table(const void* x, const int* tokens, const int* table, const void* w_gu, int il,
                 const void* w_down, void* h, float* y, int n, int D, int F, int top, int vocab, int n_experts,
                 int accumulate, int dtype, int* status, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (D <= 0 || F <= 0 || top <= 0 || vocab <= 0 || n_experts <= 0 || il < 0 || (il > 0 && F % il)) return ZK_EINVAL;
  if (dtype == ZK_F32)
    return launch_moe<float>(x, tokens, table, w_gu, il, w_down, h, y, n, D, F, top, vocab, n_experts, accumulate, status, nullptr, 0, stream);
  if (dtype == ZK_BF16)
    return launch_moe<bf16>(x, tokens, table, w_gu, il, w_down, h, y, n, D, F, top, vocab, n_experts, accumulate, status, nullptr, 0, stream);
  return ZK_EINVAL;
}

// The same with the experts a router chose: route_ids [n, top] int32 and route_w [n, top] float32 (the weight of
// each), y_t = sum_k route_w[t, k] * Expert[route_ids[t, k]](x_t), added in the order of k.  Ids n_experts ..
// n_experts + n_ident - 1 are identity experts: Expert(x_t) = x_t.
int zk_moe_routed(const void* x, const int* route_ids, const float* route_w, const void* w_gu, int il, const void* w_down,
                  void* h, float* y, int n, int D, int F, int top, int n_experts, int accumulate, int dtype, int* status,
                  int n_ident, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (D <= 0 || F <= 0 || top <= 0 || n_experts <= 0 || n_ident < 0 || il < 0 || (il > 0 && F % il) || !route_ids || !route_w) return ZK_EINVAL;
  if (dtype == ZK_F32)
    return launch_moe<float>(x, nullptr, route_ids, w_gu, il, w_down, h, y, n, D, F, top, 1, n_experts, accumulate, status, route_w, n_ident, stream);
  if (dtype == ZK_BF16)
    return launch_moe<bf16>(x, nullptr, route_ids, w_gu, il, w_down, h, y, n, D, F, top, 1, n_experts, accumulate, status, route_w, n_ident, stream);
  return ZK_EINVAL;
}

// Router: z = W x_t in float32 (W [E, D] float32, x in the run dtype), s = softmax(z) over all experts, the `top`
// largest s (ties: the lower index) are chosen and weighed s / (sum of the chosen + 1e-20).  With `correction` [E] the
// choice goes by s + correction; the weights are made of s alone.
int zk_moe_router(const void* x, const float* w_router, int* route_ids, float* route_w, int n, int D, int E, int top,
                  int dtype, const float* correction, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (D <= 0 || E <= 0 || top <= 0 || top > E || E > MOE_ROUTER_MAX_EXPERTS) return ZK_EINVAL;
  const size_t smem = sizeof(float) * ((size_t)D + 2 * (size_t)E);
  if (smem > 200 * 1024) return ZK_EINVAL;
#define ZK_ROUTER(T)                                                                                                 \
  do {                                                                                                               \
    auto kern = moe_router_kernel<T>;                                                                                \
    if (smem > 48 * 1024) {                                                                                          \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
      if (e != cudaSuccess) return (int)e;                                                                           \
    }                                                                                                                \
    return zk_launch_dependent(kern, dim3(n), dim3(MOE_WARPS * 32), smem, stream, (const T*)x, w_router, route_ids,  \
                               route_w, D, E, top, correction);                                                      \
  } while (0)
  if (dtype == ZK_F32) ZK_ROUTER(float);
  if (dtype == ZK_BF16) ZK_ROUTER(bf16);
#undef ZK_ROUTER
  return ZK_EINVAL;
}

// The device's own sort of (token, k) pairs by expert, as moe_expert_rows_kernel describes it.
int zk_moe_expert_rows(const int* ids, int P, int E, int top, int tile, int cap, int* row_token, int* pair_row,
                       int* tile_group, int n_ident, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (E <= 0 || E > 4096 || top <= 0 || tile <= 0 || cap % tile || cap < (P / tile + E) * tile) return ZK_EINVAL;
  return zk_launch_dependent(moe_expert_rows_kernel, dim3(1), dim3(1024), sizeof(int) * 2 * (size_t)E, stream, ids, P, E,
                             top, tile, cap, row_token, pair_row, tile_group, n_ident);
}

// xg[r, :] = x[row_token[r], :] for r < n_rows, zeros where row_token[r] < 0 (rows in the run dtype, D elements).
int zk_moe_gather(const void* x, const int* row_token, void* xg, int n_rows, int D, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (D <= 0) return ZK_EINVAL;
  const int threads = 128;
  if (dtype == ZK_F32)
    return zk_launch_dependent(moe_gather_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, (const float*)x, row_token, (float*)xg, D);
  if (dtype == ZK_BF16)
    return zk_launch_dependent(moe_gather_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, (const bf16*)x, row_token, (bf16*)xg, D);
  return ZK_EINVAL;
}

// out[t, :] (=|+=) (1/top) * sum_k y[pair_row[t * top + k], :], float32, added in the order of k.
int zk_moe_combine(const float* y, const int* pair_row, float* out, int n, int D, int top, int accumulate,
                   const float* route_w, const void* x_ident, int x_dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (D <= 0 || top <= 0) return ZK_EINVAL;
  return zk_launch_dependent(moe_combine_kernel, dim3(n), dim3(128), 0, stream, y, pair_row, out, D, top, accumulate, route_w,
                             x_ident, x_dtype == ZK_BF16 ? 1 : 0);
}

}  // extern "C"
