// Gated linear recurrence with a matrix state per head (HGRN2): per head a state S [d, e],
//
//     S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T,        o_t = S_t^T q_t,
//
// f_t in (lower, 1) the forget gate per head and channel; 1 - f_t is the share of v_t that enters the state
// (no key projection), q_t = silu(.), v_t plain.  A row of `qfv` holds the three projections of a token,
// [q (H*d) | f (H*d) | v (H*e)], float32 as the contraction left them; hgrn2_gates_kernel turns the first
// two parts, in place, into silu(q) and the gate f = lower + (1 - lower) * sigmoid(z_f + bias), once for
// all the blocks of the recurrence that read them.  Everything here is float32: gate, state, sums.
//
// One kernel serves prompt steps and single-token steps.  A block owns one (sequence, head, 32 value columns)
// and walks the sequence's tokens in order, from the state the step before left in `state[slot]` to the
// state it leaves there.  Its eight warps split the d channels: warp w keeps rows [w*DPT, (w+1)*DPT) of the
// 32 columns of S in registers (lane = column, so the state is read and written in whole lines), adds up its
// part of o_t = sum_i S_t[i, c] q_t[i], and the parts of sixteen tokens at a time meet in shared memory, where
// warp w sums those of tokens w and w + 8 in the order of the warps.  q and f of the next sixteen tokens are fetched into
// registers while the current sixteen are worked on, and go into the other half of a double buffer.  The order of every sum is fixed by the layout alone, so a
// sequence cut into steps gives the same bits as the whole.
//
// The same kernel runs the recurrence of a retention layer (its KEYED form): a key projection in place of the gate and
// one fixed decay per head, S_t = decay_h S_{t-1} + k_t v_t^T; retention_prepare_kernel rotates q and k and scales k first.
#include "common.cuh"
#include <math.h>

#define HG_R 8             // warps of a block, each with a stretch of the d channels
#define HG_MAX_D 512

// In place on the rows of qfv: q <- silu(q), f <- lower + (1 - lower) * sigmoid(f + bias); v is left alone.
__global__ void hgrn2_gates_kernel(float* __restrict__ qfv, int ld, const float* __restrict__ f_bias,
                                   const float* __restrict__ lower, int n, int gate_dim) {
  zk_let_next_start();
  zk_wait_prior();
  const size_t total = (size_t)n * gate_dim;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / gate_dim;
    const int i = (int)(idx - t * gate_dim);
    float* row = qfv + t * ld;
    const float zq = row[i], zf = row[gate_dim + i] + f_bias[i], lo = lower[i];
    row[i] = zq / (1.0f + expf(-zq));
    row[gate_dim + i] = lo + (1.0f - lo) * (1.0f / (1.0f + expf(-zf)));
  }
}

// What a retention layer does to its projections before the recurrence, in place on the float32 rows [q (H*d) | k (H*d)
// | ...]: the first n_rot entries of every q and k head are rotated by the token's position (entry i pairs with entry
// i + n_rot/2, angle = float(pos) * inv_freq[i]; inv_freq null = no rotation), then k is multiplied by key_scale.
// Block (t, y) takes `slots_per_block` of token t's 2H heads: the cosines and sines of the position are computed once per
// block (with many tokens one block serves all 2H heads; with few, the heads are spread over more blocks).
__global__ void __launch_bounds__(256)
    retention_prepare_kernel(float* __restrict__ qk, int ld, const float* __restrict__ inv_freq, int n_rot, float key_scale,
                             const int* __restrict__ tok_pos, int H, int d, int slots_per_block) {
  __shared__ float cs[HG_MAX_D / 2], sn[HG_MAX_D / 2];
  zk_let_next_start();
  zk_wait_prior();
  const int t = blockIdx.x;
  const int half = inv_freq ? n_rot >> 1 : 0;
  const float pos = (float)tok_pos[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float ang = pos * inv_freq[i];
    cs[i] = cosf(ang);
    sn[i] = sinf(ang);
  }
  __syncthreads();
  const int per_head = d - half;                      // work items of a head: its pairs, then its unrotated entries
  float* row = qk + (size_t)t * ld;
  const int s0 = blockIdx.y * slots_per_block, s_here = min(2 * H, s0 + slots_per_block) - s0;
  for (int idx = threadIdx.x; idx < s_here * per_head; idx += blockDim.x) {
    const int s = s0 + idx / per_head, i = idx % per_head;      // head slot: the H query heads, then the H key heads
    float* head = row + (size_t)s * d;
    const float mul = s >= H ? key_scale : 1.0f;
    if (i < half) {
      const float c = cs[i], sv = sn[i];
      const float u = head[i], v = head[i + half];
      head[i] = (u * c - v * sv) * mul;
      head[i + half] = (v * c + u * sv) * mul;
    } else if (s >= H) {
      head[i + half] *= mul;
    }
  }
}

// DPT: channels per warp; TT: tokens staged at once (sixteen, or eight or four where more do not fit shared memory).
// KEYED: the recurrence of a retention layer instead, S_t = decay_h S_{t-1} + k_t v_t^T with one fixed decay per head
// (`decay` [H]); the row's second part then holds the keys k_t in place of the gates.
template <int DPT, int TT, bool KEYED>
__global__ void __launch_bounds__(HG_R * 32)
    hgrn2_scan_kernel(const float* __restrict__ qfv, int ld, float* __restrict__ state, long long state_stride,
                      float* __restrict__ o, const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int H, int d,
                      int e, const float* __restrict__ decay) {
  constexpr int DM = HG_R * DPT;                                     // channels the block covers, >= d
  constexpr int NL = (TT * DM + HG_R * 32 - 1) / (HG_R * 32);     // q (and f) values a thread fetches per group of tokens
  __shared__ __align__(16) float qs[2][TT][DM];
  __shared__ __align__(16) float fs[2][TT][DM];
  __shared__ float part[TT][HG_R][32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = blockIdx.x, h = blockIdx.y;
  const int c = blockIdx.z * 32 + lane;
  const bool col = c < e;
  const int row0 = warp * DPT;
  // channels beyond d: q = 0 and f = 0 for good, so they add nothing
  if (d < DM) {
    for (int i = tid; i < 2 * TT * DM; i += HG_R * 32) {
      (&qs[0][0][0])[i] = 0.f;
      (&fs[0][0][0])[i] = 0.f;
    }
    __syncthreads();
  }
  zk_wait_prior();   // qfv is the kernel before's result
  const int t0 = cu_q[b], t1 = cu_q[b + 1];
  const float dk = KEYED ? decay[h] : 0.f;
  float* st = state + (size_t)seq_slot[b] * state_stride + (size_t)h * d * e;
  float S[DPT];
#pragma unroll
  for (int k = 0; k < DPT; ++k) S[k] = (col && row0 + k < d) ? st[(size_t)(row0 + k) * e + c] : 0.f;

  const int off_f = H * d, off_v = 2 * H * d;
  float rq[NL], rf[NL], v_cur[TT], v_next[TT];
  // where a thread's n-th value of a group comes from (relative to the group's first row) and goes to
  int src[NL], dst[NL];
#pragma unroll
  for (int n = 0; n < NL; ++n) {
    const int idx = tid + n * HG_R * 32;
    const int tt = idx / d, i = idx - tt * d;
    src[n] = tt < TT ? tt * ld + h * d + i : -1;
    dst[n] = tt * DM + i;
  }
  auto fetch = [&](int tb) {
    const int nt = min(TT, t1 - tb);
    const float* base = qfv + (size_t)tb * ld;
#pragma unroll
    for (int n = 0; n < NL; ++n) {
      const bool ok = src[n] >= 0 && tid + n * HG_R * 32 < nt * d;
      rq[n] = ok ? base[src[n]] : 0.f;
      rf[n] = ok ? base[src[n] + off_f] : 0.f;
    }
#pragma unroll
    for (int tt = 0; tt < TT; ++tt)
      v_next[tt] = (col && tt < nt) ? base[(size_t)tt * ld + off_v + h * e + c] : 0.f;
  };
  auto stage = [&](int buf, int tb) {
    const int nt = min(TT, t1 - tb);
#pragma unroll
    for (int n = 0; n < NL; ++n) {
      if (src[n] >= 0 && tid + n * HG_R * 32 < nt * d) {
        (&qs[buf][0][0])[dst[n]] = rq[n];
        (&fs[buf][0][0])[dst[n]] = rf[n];
      }
    }
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) v_cur[tt] = v_next[tt];
  };

  if (t0 < t1) {
    fetch(t0);
    stage(0, t0);
  }
  __syncthreads();
  int buf = 0;
  for (int tb = t0; tb < t1; tb += TT, buf ^= 1) {
    const int nt = min(TT, t1 - tb);
    const bool more = tb + TT < t1;
    if (more) fetch(tb + TT);       // under way while this group is worked on
    auto token = [&](int tt) {
      const float v = v_cur[tt];
      float acc = 0.f;
      if constexpr (DPT % 4 == 0) {
#pragma unroll
        for (int k4 = 0; k4 < DPT; k4 += 4) {
          const float4 f4 = *reinterpret_cast<const float4*>(&fs[buf][tt][row0 + k4]);
          const float4 q4 = *reinterpret_cast<const float4*>(&qs[buf][tt][row0 + k4]);
          const float ff[4] = {f4.x, f4.y, f4.z, f4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (KEYED) S[k4 + j] = fmaf(dk, S[k4 + j], ff[j] * v);               // decay S + k v
            else S[k4 + j] = fmaf(ff[j], S[k4 + j], fmaf(-ff[j], v, v));        // f S + (1 - f) v
            acc = fmaf(S[k4 + j], qq[j], acc);
          }
        }
      } else {
#pragma unroll
        for (int k = 0; k < DPT; ++k) {
          const float f = fs[buf][tt][row0 + k];
          if (KEYED) S[k] = fmaf(dk, S[k], f * v);
          else S[k] = fmaf(f, S[k], fmaf(-f, v, v));
          acc = fmaf(S[k], qs[buf][tt][row0 + k], acc);
        }
      }
      part[tt][warp][lane] = acc;
    };
    if (nt == TT) {          // a whole group: no branch between the tokens, so their loads and sums interleave
#pragma unroll
      for (int tt = 0; tt < TT; ++tt) token(tt);
    } else {
#pragma unroll
      for (int tt = 0; tt < TT; ++tt)
        if (tt < nt) token(tt);
    }
    __syncthreads();
#pragma unroll
    for (int tt = warp; tt < TT; tt += HG_R) {
      if (tt < nt && col) {
        float sum = 0.f;
#pragma unroll
        for (int r = 0; r < HG_R; ++r) sum += part[tt][r][lane];
        o[(size_t)(tb + tt) * H * e + (size_t)h * e + c] = sum;
      }
    }
    if (more) stage(buf ^ 1, tb + TT);
    __syncthreads();
  }
  // The kernel behind this one may start only now: a block that waits for this long kernel to end would hold
  // an SM's issue slots against it (measured: the recurrence ran at half its speed with the release at its top).
  zk_let_next_start();
  if (col) {
#pragma unroll
    for (int k = 0; k < DPT; ++k)
      if (row0 + k < d) st[(size_t)(row0 + k) * e + c] = S[k];
  }
}

extern "C" {

int zk_hgrn2_max_dim() { return HG_MAX_D; }

// qfv float32 [n, >= 2*H*d + H*e] with rows `ld` floats apart, whose q and f parts are REPLACED by silu(q) and the
// gate; f_bias, lower float32 [H*d]; state float32, a
// slot's [H, d, e] block `state_stride` floats after the one before; o float32 [n, H*e]; cu_q [n_seqs + 1],
// seq_slot [n_seqs].
int zk_hgrn2_scan(float* qfv, int ld, const float* f_bias, const float* lower, float* state, long long state_stride,
                  float* o, const int* cu_q, const int* seq_slot, int n, int n_seqs, int H, int d, int e, cudaStream_t stream) {
  if (n_seqs <= 0 || n <= 0) return 0;
  if (H <= 0 || d <= 0 || e <= 0 || d > HG_MAX_D || ld < 2 * H * d + H * e || !f_bias || !lower) return ZK_EINVAL;
  {
    const size_t total = (size_t)n * H * d;
    const int threads = 256;
    const size_t want = (total + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    const int rc = zk_launch_dependent(hgrn2_gates_kernel, dim3(blocks), dim3(threads), 0, stream, qfv, ld, f_bias, lower, n, H * d);
    if (rc != 0) return rc;
  }
  dim3 grid(n_seqs, H, (e + 31) / 32);
#define ZK_HG(DP)                                                                                                    \
  return zk_launch_dependent(hgrn2_scan_kernel<DP, (DP > 32 ? 4 : (DP > 16 ? 8 : 16)), false>, grid, dim3(HG_R * 32), 0, stream, (const float*)qfv, ld, \
                             state, state_stride, o, cu_q, seq_slot, H, d, e, (const float*)nullptr)
  const int dpt = (d + HG_R - 1) / HG_R;
  if (dpt <= 1) ZK_HG(1);
  if (dpt <= 2) ZK_HG(2);
  if (dpt <= 4) ZK_HG(4);
  if (dpt <= 8) ZK_HG(8);
  if (dpt <= 16) ZK_HG(16);
  if (dpt <= 32) ZK_HG(32);
  ZK_HG(64);
#undef ZK_HG
}

// Retention: per head S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t.  qkv float32 [n, >= 2*H*d + H*e] with rows `ld`
// floats apart, [q | k | v | ...] as the projections gave them; q and k are REPLACED by their rotated forms (k also
// times key_scale).  decay float32 [H]; inv_freq float32 [n_rot / 2] or null; tok_pos [n]; state, o, cu_q, seq_slot as for
// zk_hgrn2_scan.
int zk_retention_scan(float* qkv, int ld, const float* decay, const float* inv_freq, int n_rot, float key_scale,
                      const int* tok_pos, float* state, long long state_stride, float* o, const int* cu_q,
                      const int* seq_slot, int n, int n_seqs, int H, int d, int e, cudaStream_t stream) {
  if (n_seqs <= 0 || n <= 0) return 0;
  if (H <= 0 || d <= 0 || e <= 0 || d > HG_MAX_D || ld < 2 * H * d + H * e || !decay || !tok_pos) return ZK_EINVAL;
  if (inv_freq && (n_rot <= 0 || (n_rot & 1) || n_rot > d)) return ZK_EINVAL;
  if (inv_freq || key_scale != 1.0f) {
    const int per = n >= 256 ? 2 * H : (2 * H + 7) / 8;       // head slots a block takes
    const int rc = zk_launch_dependent(retention_prepare_kernel, dim3(n, (2 * H + per - 1) / per), dim3(256), 0, stream, qkv, ld,
                                       inv_freq, n_rot, key_scale, tok_pos, H, d, per);
    if (rc != 0) return rc;
  }
  dim3 grid(n_seqs, H, (e + 31) / 32);
#define ZK_RT(DP)                                                                                                    \
  return zk_launch_dependent(hgrn2_scan_kernel<DP, (DP > 32 ? 4 : (DP > 16 ? 8 : 16)), true>, grid, dim3(HG_R * 32), 0, stream, (const float*)qkv, ld, \
                             state, state_stride, o, cu_q, seq_slot, H, d, e, decay)
  const int dpt = (d + HG_R - 1) / HG_R;
  if (dpt <= 1) ZK_RT(1);
  if (dpt <= 2) ZK_RT(2);
  if (dpt <= 4) ZK_RT(4);
  if (dpt <= 8) ZK_RT(8);
  if (dpt <= 16) ZK_RT(16);
  if (dpt <= 32) ZK_RT(32);
  ZK_RT(64);
#undef ZK_RT
}

}  // extern "C"
