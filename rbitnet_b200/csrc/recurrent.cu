// Recurrent mixers: what runs from token to token of a sequence, with the state kept per cache slot.
//
//   causal convolution  u_t[c] = b[c] + sum_j taps[c][j] * x_(t-(K-1-j))[c]      (K taps, the last is the current token's)
//   gated linear unit   r = sigmoid(g_r), i = sigmoid(g_i), a = exp(-c * r * softplus(lam)),
//                       S_t = a S_(t-1) + sqrt(1 - a^2) * i * u_t ;   out = S_t * gelu_tanh(y_t)
//   matrix memory       m_t = max(f + m_(t-1), i);  C_t = e^(f + m_(t-1) - m_t) C_(t-1) + e^(i - m_t) k v^T;
//                       n_t likewise with k alone;  o = C_t^T q / (max(|n_t . q|, e^(-m_t)) + floor)
//
// A step brings, per sequence, a run of consecutive rows (its next tokens); seq_first / seq_count
// name each run, and the state of the run's slot is read at its start and written back at its end,
// so a prompt may arrive whole, in portions or token by token.  States, gates, decays, exponentials
// and sums are float32 whatever the dtype of the projections.
#include "rb_common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf_(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplusf_(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }
__device__ __forceinline__ float gelu_tanh_(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// ---------------------------------------------------------------- causal convolution
// x: rows [T, ldx] of the projections' dtype, the convolved channels at column x_off; the bias x_bias
// is added to every input before the taps.  tail: [n_slots, K, C] float32, a ring by position: the input
// (with its bias) of position q of the slot's sequence is kept at row q mod K, so that writing a position
// never touches one of the K-1 positions before it, which the same step may still be reading; zeros at
// the start of a sequence.  tok_first: row of the first token of the row's run (null: every row is its own run).
constexpr int CONV_TOKENS = 8;
template <typename TI>
__global__ void conv_causal_kernel(float* __restrict__ u, const TI* __restrict__ x, int64_t ldx, int x_off,
                                   const float* __restrict__ x_bias, const float* __restrict__ taps,
                                   const float* __restrict__ conv_bias, const float* __restrict__ tail,
                                   const int* __restrict__ tok_first, const int* __restrict__ tok_slot,
                                   const int* __restrict__ tok_pos, int n_tokens, int C, int K, int silu, int per_block) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  // with many rows a block takes per_block neighbouring rows in turn: the earlier rows a row reads are then mostly in
  // the SM's cache
  for (int t = blockIdx.x * per_block; t < min(n_tokens, (int)(blockIdx.x + 1) * per_block); ++t) {
  const int first = tok_first != nullptr ? tok_first[t] : t;
  const int slot = tok_slot[t], pos = tok_pos[t];
  const int j = t - first;                      // rows of this run before this one
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float acc = conv_bias != nullptr ? conv_bias[c] : 0.f;
    const float xb = x_bias != nullptr ? x_bias[c] : 0.f;
    for (int d = 0; d < K; ++d) {               // d tokens back
      float v;
      if (d <= j) v = rb_to_float<TI>(x[(int64_t)(t - d) * ldx + x_off + c]) + xb;
      else if (pos - d < 0) v = 0.f;
      else v = tail[((int64_t)slot * K + (pos - d) % K) * C + c];
      acc = fmaf(taps[(int64_t)c * K + (K - 1 - d)], v, acc);
    }
    u[(int64_t)t * C + c] = silu ? acc * sigmoidf_(acc) : acc;
  }
  }
}

// The ring of a convolution's last inputs moves on to the end of every run: the inputs (with their bias) of the
// run's last K-1 positions go to their rows.  For a mixer whose recurrence kernel does not do this itself.
template <typename TI>
__global__ void conv_tail_kernel(float* __restrict__ tail, const TI* __restrict__ x, int64_t ldx, int x_off,
                                 const float* __restrict__ x_bias, const int* __restrict__ seq_first,
                                 const int* __restrict__ seq_count, const int* __restrict__ tok_slot,
                                 const int* __restrict__ tok_pos, int C, int K) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int first = seq_first != nullptr ? seq_first[blockIdx.x] : blockIdx.x;
  const int n = seq_count != nullptr ? seq_count[blockIdx.x] : 1;
  const int slot = tok_slot[first], pos0 = tok_pos[first];
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    const float xb = x_bias != nullptr ? x_bias[c] : 0.f;
    for (int back = 0; back < K - 1 && back < n; ++back) {
      const int q = pos0 + n - 1 - back;
      tail[((int64_t)slot * K + q % K) * C + c] = rb_to_float<TI>(x[(int64_t)(first + n - 1 - back) * ldx + x_off + c]) + xb;
    }
  }
}

// ---------------------------------------------------------------- gated linear recurrent unit
// One thread per (run, channel).  gates: [T, blocks, 2, Wb] float32 pre-activations (recurrence gate,
// input gate) of the channel's block.  Also moves the convolution's tail on to the end of the run.
template <typename TI, typename TO>
__global__ void __launch_bounds__(64) gated_scan_kernel(
    TO* __restrict__ out, const float* __restrict__ u, const float* __restrict__ gates, const float* __restrict__ gate_r_bias,
    const float* __restrict__ gate_i_bias, const float* __restrict__ lam, float decay_scale, const TI* __restrict__ xy,
    int64_t ldxy, int x_off, int y_off, const float* __restrict__ x_bias, const float* __restrict__ y_bias,
    float* __restrict__ state, float* __restrict__ tail, const int* __restrict__ seq_first,
    const int* __restrict__ seq_count, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, int W, int Wb, int K) {
  rb_pdl_launch_dependents();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= W) return;
  const float sp = decay_scale * softplusf_(lam[c]);
  const float br = gate_r_bias[c], bi = gate_i_bias[c];
  const float yb = y_bias != nullptr ? y_bias[c] : 0.f;
  const float xb = x_bias != nullptr ? x_bias[c] : 0.f;
  const int blk = c / Wb, o = c % Wb;
  rb_pdl_wait();
  const int first = seq_first != nullptr ? seq_first[blockIdx.x] : blockIdx.x;
  const int n = seq_count != nullptr ? seq_count[blockIdx.x] : 1;
  const int slot = tok_slot[first];
  float S = state[(int64_t)slot * W + c];
  for (int t = first; t < first + n; ++t) {
    const float* g = gates + ((int64_t)t * (W / Wb) + blk) * 2 * Wb;
    const float r = sigmoidf_(g[o] + br);
    const float i = sigmoidf_(g[Wb + o] + bi);
    const float a = expf(-sp * r);
    S = fmaf(a, S, sqrtf(1.0f - a * a) * i * u[(int64_t)t * W + c]);
    const float y = gelu_tanh_(rb_to_float<TI>(xy[(int64_t)t * ldxy + y_off + c]) + yb);
    out[(int64_t)t * W + c] = rb_from_float<TO>(S * y);
  }
  state[(int64_t)slot * W + c] = S;
  // the run's last inputs go to their rows of the ring
  if (K > 1) {
    const int pos0 = tok_pos[first];
    for (int back = 0; back < K - 1 && back < n; ++back) {
      const int q = pos0 + n - 1 - back;
      tail[((int64_t)slot * K + q % K) * W + c] = rb_to_float<TI>(xy[(int64_t)(first + n - 1 - back) * ldxy + x_off + c]) + xb;
    }
  }
}

// ---- long runs: the gates become decays and drives in one pass over all rows, then a scan in chunks of time
// a = exp(-c softplus(lam) sigmoid(g_r + b_r)) replaces g_r and b = sqrt(1 - a^2) sigmoid(g_i + b_i) u replaces g_i, in place.
__global__ void gate_prepare_kernel(float* __restrict__ gates, const float* __restrict__ u, const float* __restrict__ gate_r_bias,
                                    const float* __restrict__ gate_i_bias, const float* __restrict__ lam, float decay_scale,
                                    int64_t n, int W, int Wb) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / W;
    const int c = (int)(i % W);
    const int blk = c / Wb, o = c % Wb;
    float* g = gates + (t * (W / Wb) + blk) * 2 * Wb;
    const float r = sigmoidf_(g[o] + gate_r_bias[c]);
    const float in = sigmoidf_(g[Wb + o] + gate_i_bias[c]);
    const float a = expf(-decay_scale * softplusf_(lam[c]) * r);
    g[o] = a;
    g[Wb + o] = sqrtf(1.0f - a * a) * in * u[i];
  }
}

// One block per (run, 32 channels): 32 lanes are 32 channels (rows of the inputs are read 128 bytes at a time),
// the block's 32 warps are 32 chunks of the run's time.  Every warp first folds its chunk into (A, B) with
// S_end = A S_begin + B, the chunks' pairs are chained in shared memory, and a second pass over the chunk
// writes S_t * gelu_tanh(y_t).
constexpr int SCAN_CH = 32, SCAN_CHUNKS = 32;
template <typename TI, typename TO>
__global__ void __launch_bounds__(SCAN_CH * SCAN_CHUNKS) gated_scan_chunked_kernel(
    TO* __restrict__ out, const float* __restrict__ ab, const TI* __restrict__ xy, int64_t ldxy, int x_off, int y_off,
    const float* __restrict__ x_bias, const float* __restrict__ y_bias, float* __restrict__ state, float* __restrict__ tail,
    const int* __restrict__ seq_first, const int* __restrict__ seq_count, const int* __restrict__ tok_slot,
    const int* __restrict__ tok_pos, int W, int Wb, int K) {
  rb_pdl_launch_dependents();
  __shared__ float sA[SCAN_CHUNKS][SCAN_CH], sB[SCAN_CHUNKS][SCAN_CH];
  const int lane = threadIdx.x & 31, chunk = threadIdx.x >> 5;
  const int c = blockIdx.y * SCAN_CH + lane;
  const bool live = c < W;
  const int cc = live ? c : 0;
  const float yb = y_bias != nullptr ? y_bias[cc] : 0.f;
  const float xb = x_bias != nullptr ? x_bias[cc] : 0.f;
  const int blk = cc / Wb, o = cc % Wb;
  rb_pdl_wait();
  const int first = seq_first[blockIdx.x], n = seq_count[blockIdx.x];
  const int slot = tok_slot[first];
  const int L = (n + SCAN_CHUNKS - 1) / SCAN_CHUNKS;
  const int t0 = first + min(n, chunk * L), t1 = first + min(n, (chunk + 1) * L);
  const int nb = W / Wb;
  float A = 1.f, B = 0.f;
  for (int t = t0; t < t1; ++t) {
    const float* g = ab + ((int64_t)t * nb + blk) * 2 * Wb;
    const float a = g[o], b = g[Wb + o];
    B = fmaf(a, B, b);
    A *= a;
  }
  sA[chunk][lane] = A;
  sB[chunk][lane] = B;
  __syncthreads();
  float S = live ? state[(int64_t)slot * W + cc] : 0.f;
  for (int k = 0; k < chunk; ++k) S = fmaf(sA[k][lane], S, sB[k][lane]);
  for (int t = t0; t < t1; ++t) {
    const float* g = ab + ((int64_t)t * nb + blk) * 2 * Wb;
    S = fmaf(g[o], S, g[Wb + o]);
    const float y = gelu_tanh_(rb_to_float<TI>(xy[(int64_t)t * ldxy + y_off + cc]) + yb);
    if (live) out[(int64_t)t * W + cc] = rb_from_float<TO>(S * y);
  }
  if (!live) return;
  if (chunk == SCAN_CHUNKS - 1) state[(int64_t)slot * W + cc] = S;       // the last chunk ends where the run ends
  if (chunk == 0 && K > 1) {
    const int pos0 = tok_pos[first];
    for (int back = 0; back < K - 1 && back < n; ++back) {
      const int q = pos0 + n - 1 - back;
      tail[((int64_t)slot * K + q % K) * W + cc] = rb_to_float<TI>(xy[(int64_t)(first + n - 1 - back) * ldxy + x_off + cc]) + xb;
    }
  }
}

// ---- a few rows, each its own sequence (a decode step): convolution, gates, recurrence and output in one kernel
// One block per (block of the gates' matrices, STEP_CH of its channels), one warp per channel.  The block convolves all
// Wb channels of the gates' block for every row (the gates of a channel read them all); a warp reads its channel's two
// rows of weights once, by lanes and eight loads at a time, for all rows' sums; lane t then finishes row t.
constexpr int STEP_CH = 8, STEP_MAX_ROWS = 16;
template <typename TI, typename TO>
__global__ void __launch_bounds__(32 * STEP_CH) gated_step_kernel(
    TO* __restrict__ out, const TI* __restrict__ xy, int64_t ldxy, int x_off, int y_off, const float* __restrict__ x_bias,
    const float* __restrict__ y_bias, const float* __restrict__ taps, const float* __restrict__ conv_bias,
    const float* __restrict__ w_gates, const float* __restrict__ gate_r_bias, const float* __restrict__ gate_i_bias,
    const float* __restrict__ lam, float decay_scale, float* __restrict__ state, float* __restrict__ tail,
    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, int T, int W, int Wb, int K) {
  rb_pdl_launch_dependents();
  extern __shared__ float s_u[];                 // [T][Wb]
  const int b = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int o = blockIdx.y * STEP_CH + warp;      // this warp's channel within the block
  const bool has = o < Wb;
  const int c = b * Wb + (has ? o : 0);
  // the channel's two rows of weights do not depend on the kernel before: the first eight loads start now
  const float* wr = w_gates + ((int64_t)b * 2 * Wb + (has ? o : 0)) * Wb;
  const float* wi = wr + (int64_t)Wb * Wb;
  float w0[4], w1[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = lane + 32 * j;
    w0[j] = i < Wb ? wr[i] : 0.f;
    w1[j] = i < Wb ? wi[i] : 0.f;
  }
  const float sp = decay_scale * softplusf_(lam[c]);
  const float br = gate_r_bias[c], bi = gate_i_bias[c];
  rb_pdl_wait();
  for (int idx = threadIdx.x; idx < T * Wb; idx += blockDim.x) {
    const int t = idx / Wb, i = idx - t * Wb, cc = b * Wb + i;
    const int slot = tok_slot[t], pos = tok_pos[t];
    float acc = conv_bias != nullptr ? conv_bias[cc] : 0.f;
    for (int d = 0; d < K; ++d) {
      float v;
      if (d == 0) v = rb_to_float<TI>(xy[(int64_t)t * ldxy + x_off + cc]) + (x_bias != nullptr ? x_bias[cc] : 0.f);
      else if (pos - d < 0) v = 0.f;
      else v = tail[((int64_t)slot * K + (pos - d) % K) * W + cc];
      acc = fmaf(taps[(int64_t)cc * K + (K - 1 - d)], v, acc);
    }
    s_u[idx] = acc;
  }
  __syncthreads();
  float ar[STEP_MAX_ROWS], ai[STEP_MAX_ROWS];
#pragma unroll
  for (int t = 0; t < STEP_MAX_ROWS; ++t) ar[t] = ai[t] = 0.f;
  for (int i0 = 0; i0 < Wb; i0 += 128) {
    if (i0 > 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = i0 + lane + 32 * j;
        w0[j] = i < Wb ? wr[i] : 0.f;
        w1[j] = i < Wb ? wi[i] : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = i0 + lane + 32 * j;
      if (i < Wb) {
#pragma unroll
        for (int t = 0; t < STEP_MAX_ROWS; ++t)
          if (t < T) {
            const float u = s_u[t * Wb + i];
            ar[t] = fmaf(w0[j], u, ar[t]);
            ai[t] = fmaf(w1[j], u, ai[t]);
          }
      }
    }
  }
  float gr = 0.f, gi = 0.f;                       // lane t keeps row t's sums
#pragma unroll
  for (int t = 0; t < STEP_MAX_ROWS; ++t) {
    if (t < T) {
      const float a = rb_warp_sum(ar[t]), bsum = rb_warp_sum(ai[t]);
      if (lane == t) { gr = a; gi = bsum; }
    }
  }
  if (!has || lane >= T) return;
  const int t = lane;
  const int slot = tok_slot[t], pos = tok_pos[t];
  const float r = sigmoidf_(gr + br), in = sigmoidf_(gi + bi);
  const float a = expf(-sp * r);
  float S = state[(int64_t)slot * W + c];
  S = fmaf(a, S, sqrtf(1.0f - a * a) * in * s_u[t * Wb + o]);
  state[(int64_t)slot * W + c] = S;
  const float y = gelu_tanh_(rb_to_float<TI>(xy[(int64_t)t * ldxy + y_off + c]) + (y_bias != nullptr ? y_bias[c] : 0.f));
  out[(int64_t)t * W + c] = rb_from_float<TO>(S * y);
  if (K > 1)
    tail[((int64_t)slot * K + pos % K) * W + c] = rb_to_float<TI>(xy[(int64_t)t * ldxy + x_off + c]) + (x_bias != nullptr ? x_bias[c] : 0.f);
}

// ---------------------------------------------------------------- matrix memory
// One block per (run, head, tile of value columns).  A thread owns one value column j and every P-th
// row d of the memory (R rows at most), so a token costs it 2 R multiply-adds and the sums over d are
// finished with log2(P) shuffles.  Rows of the projections: [q (H D) | k (H D) | v (H Dv) | ... ], gate
// pre-activations at columns i_off + h and f_off + h.  Tokens are staged TT at a time in shared memory.
constexpr int MM_TT = 16;

__device__ __forceinline__ void cp_async_f32(float* smem_dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_f32x4(float* smem_dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// The memory of a (slot, head) is kept as [value column][row] (the kernel's own layout; nobody else reads it).
// One block per (run, head, tile of value columns); blockDim / P columns per block.  A thread owns one value
// column j and the rows d = part + P r (r < R) of the memory, so a token costs it 2 R multiply-adds for the
// memory and as many for the sums over d, which P lanes finish with shuffles, a whole tile of tokens at once.
// The projections are float32 rows [q (H D) | k (H D) | v (H Dv) | ...], gate pre-activations at columns
// i_off + h and f_off + h.  A tile of TT tokens is copied into one of two shared buffers with cp.async while the
// tile before it is worked on (16 bytes at a time where the rows allow, vec4 != 0); rows of k and q are P R long
// in shared memory, zeros behind D, so the loop over d needs no test and its addresses are constants.
template <int P, int R>
__global__ void __launch_bounds__(128) matrix_memory_kernel(
    float* __restrict__ o_out, const float* __restrict__ proj, int64_t ld, int q_off, int k_off, int v_off, int i_off,
    int f_off, const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
    float floor_add, float* __restrict__ C_state, float* __restrict__ n_state, float* __restrict__ m_state,
    const int* __restrict__ seq_first, const int* __restrict__ seq_count, const int* __restrict__ tok_slot, int H, int D,
    int Dv, int vec4) {
  rb_pdl_launch_dependents();
  extern __shared__ __align__(16) float sm[];
  constexpr int Dp = P * R;
  const int threads = blockDim.x;
  const int cols = threads / P;
  const int cols4 = (cols + 3) & ~3;
  const int tile_floats = MM_TT * (2 * Dp + cols4 + 4);
  const int h = blockIdx.y;
  const int col = threadIdx.x / P, part = threadIdx.x % P;
  const int j = blockIdx.z * cols + col;
  const bool live = j < Dv;
  const float ib = i_bias != nullptr ? i_bias[h] : 0.f, fb = f_bias != nullptr ? f_bias[h] : 0.f;
  float* s_dec = sm + 2 * tile_floats;           // [TT][3]: decay of the memory, weight of the new pair, e^(-m)
  float* s_m = s_dec + 3 * MM_TT;                // the running maximum at the end of the tile before
  // zeros behind D in both buffers, once (the copies never write there)
  if (D < Dp) {
    for (int e = threadIdx.x; e < 2 * 2 * MM_TT * Dp; e += threads) {
      const int b = e / (2 * MM_TT * Dp), r = e % (2 * MM_TT * Dp);
      if (r % Dp >= D) sm[b * tile_floats + r] = 0.f;
    }
  }
  rb_pdl_wait();
  const int first = seq_first != nullptr ? seq_first[blockIdx.x] : blockIdx.x;
  const int n = seq_count != nullptr ? seq_count[blockIdx.x] : 1;
  const int slot = tok_slot[first];

  auto stage = [&](int t0, int buf) {
    float* s_q = sm + buf * tile_floats;         // [TT][Dp]
    float* s_k = s_q + MM_TT * Dp;               // [TT][Dp]
    float* s_v = s_k + MM_TT * Dp;               // [TT][cols4]
    float* s_g = s_v + MM_TT * cols4;            // [TT][2]: input gate, forget gate (pre-activations)
    const int nt = min(MM_TT, n - t0);
    if (vec4) {
      const int D4 = D >> 2;
      for (int e = threadIdx.x; e < nt * D4; e += threads) {
        const int tt = e / D4, d = (e - tt * D4) << 2;
        const float* row = proj + (int64_t)(first + t0 + tt) * ld + h * D + d;
        cp_async_f32x4(s_q + tt * Dp + d, row + q_off);
        cp_async_f32x4(s_k + tt * Dp + d, row + k_off);
      }
    } else {
      for (int e = threadIdx.x; e < nt * D; e += threads) {
        const int tt = e / D, d = e - tt * D;
        const float* row = proj + (int64_t)(first + t0 + tt) * ld + h * D + d;
        cp_async_f32(s_q + tt * Dp + d, row + q_off);
        cp_async_f32(s_k + tt * Dp + d, row + k_off);
      }
    }
    for (int e = threadIdx.x; e < nt * cols; e += threads) {
      const int tt = e / cols, cc = e - tt * cols;
      const int jj = blockIdx.z * cols + cc;
      if (jj < Dv) cp_async_f32(s_v + tt * cols4 + cc, proj + (int64_t)(first + t0 + tt) * ld + v_off + h * Dv + jj);
      else s_v[tt * cols4 + cc] = 0.f;
    }
    for (int tt = threadIdx.x; tt < nt; tt += threads) {
      const float* row = proj + (int64_t)(first + t0 + tt) * ld;
      cp_async_f32(s_g + 2 * tt, row + i_off + h);
      cp_async_f32(s_g + 2 * tt + 1, row + f_off + h);
    }
    cp_async_commit();
  };

  stage(0, 0);
  float Cr[R], nr[R];
  float* Cs = C_state + ((int64_t)slot * H + h) * D * Dv;
  float* ns = n_state + ((int64_t)slot * H + h) * D;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = part + P * r;
    Cr[r] = (live && d < D) ? Cs[(int64_t)j * D + d] : 0.f;      // kept [value column][row]: a column's lanes read neighbours
    nr[r] = d < D ? ns[d] : 0.f;
  }
  if (threadIdx.x == 0) *s_m = m_state[(int64_t)slot * H + h];
  int buf = 0;
  for (int t0 = 0; t0 < n; t0 += MM_TT, buf ^= 1) {
    const int nt = min(MM_TT, n - t0);
    if (t0 + MM_TT < n) {
      stage(t0 + MM_TT, buf ^ 1);        // the buffer that the tile before this one used: everybody left it at the last barrier
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* s_q = sm + buf * tile_floats;
    const float* s_k = s_q + MM_TT * Dp;
    const float* s_v = s_k + MM_TT * Dp;
    const float* s_g = s_v + MM_TT * cols4;
    // The tile's gates at once, by the first warp (lane = token).  m_t = max(f_t + m_(t-1), i_t) unrolls to
    // m_t = F_t + max(m_0, max_(s<=t)(i_s - F_s)) with F_t the sum of the tile's log forget gates up to t: a prefix
    // sum and a prefix maximum.  What the loop over tokens needs of them (e^(f + m_(t-1) - m_t), e^(i - m_t), e^(-m_t))
    // is left in shared memory, so that loop holds no exponential.
    if (threadIdx.x < 32) {
      const int tt = threadIdx.x;
      const bool on = tt < nt;
      float ig = -INFINITY, fg = 0.f;
      if (on) {
        const float ip = s_g[2 * tt] + ib, fp = s_g[2 * tt + 1] + fb;
        const float fc = cap * tanhf(fp / cap);
        ig = cap * tanhf(ip / cap);
        fg = fminf(fc, 0.f) - log1pf(expf(-fabsf(fc)));       // log sigmoid
      }
      float F = fg;
#pragma unroll
      for (int o = 1; o < MM_TT; o <<= 1) {
        const float v = __shfl_up_sync(0xffffffffu, F, o);
        if (tt >= o) F += v;
      }
      float G = ig - F;
#pragma unroll
      for (int o = 1; o < MM_TT; o <<= 1) {
        const float v = __shfl_up_sync(0xffffffffu, G, o);
        if (tt >= o) G = fmaxf(G, v);
      }
      const float m0 = *s_m;
      const float mt = F + fmaxf(m0, G);
      float mp = __shfl_up_sync(0xffffffffu, mt, 1);
      if (tt == 0) mp = m0;
      __syncwarp();
      if (on) {
        s_dec[3 * tt] = expf(fg + mp - mt);
        s_dec[3 * tt + 1] = expf(ig - mt);
        s_dec[3 * tt + 2] = expf(-mt);
        if (tt == nt - 1) *s_m = mt;
      }
    }
    __syncthreads();
    float num[MM_TT], nq[MM_TT];
    const float* kp = s_k + part;
    const float* qp = s_q + part;
#pragma unroll
    for (int tt = 0; tt < MM_TT; ++tt) {
      num[tt] = 0.f;
      nq[tt] = 0.f;
      if (tt < nt) {
        const float keep = s_dec[3 * tt], take = s_dec[3 * tt + 1];
        const float tv = take * s_v[tt * cols4 + col];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float kd = kp[tt * Dp + P * r], qd = qp[tt * Dp + P * r];
          Cr[r] = fmaf(keep, Cr[r], tv * kd);
          nr[r] = fmaf(keep, nr[r], take * kd);
          num[tt] = fmaf(Cr[r], qd, num[tt]);
          nq[tt] = fmaf(nr[r], qd, nq[tt]);
        }
      }
    }
    // the sums over a column's lanes and the divisions, for the whole tile at once: none waits for another
#pragma unroll
    for (int off = P >> 1; off > 0; off >>= 1) {
#pragma unroll
      for (int tt = 0; tt < MM_TT; ++tt) {
        num[tt] += __shfl_xor_sync(0xffffffffu, num[tt], off);
        nq[tt] += __shfl_xor_sync(0xffffffffu, nq[tt], off);
      }
    }
    if (live && part == 0) {
#pragma unroll
      for (int tt = 0; tt < MM_TT; ++tt) {
        if (tt < nt) {
          const float den = fmaxf(fabsf(nq[tt] * q_scale), s_dec[3 * tt + 2]) + floor_add;
          o_out[(int64_t)(first + t0 + tt) * H * Dv + h * Dv + j] = num[tt] * q_scale / den;
        }
      }
    }
    __syncthreads();                       // the buffer may be filled again
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = part + P * r;
    if (live && d < D) Cs[(int64_t)j * D + d] = Cr[r];
    if (blockIdx.z == 0 && col == 0 && d < D) ns[d] = nr[r];
  }
  if (blockIdx.z == 0 && threadIdx.x == 0) m_state[(int64_t)slot * H + h] = *s_m;
}

// Per (token, head): o / rms(o) over the head's Dv values, times the weight, times sigmoid(gate) (gate_silu: times
// gate * sigmoid(gate)).  One warp each.  gate: the projections' rows, at column g_off.  The weight has H * Dv
// values, or Dv values that every head uses (w_shared).
template <typename TI, typename TO>
__global__ void head_norm_gate_kernel(TO* __restrict__ out, const float* __restrict__ o, const float* __restrict__ w,
                                      const TI* __restrict__ proj, int64_t ld, int g_off, int n_rows, int H, int Dv,
                                      float eps, int w_shared, int gate_silu) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (int64_t)n_rows * H) return;
  const int t = (int)(item / H), h = (int)(item % H);
  const float* row = o + ((int64_t)t * H + h) * Dv;
  float ss = 0.f;
  for (int j = lane; j < Dv; j += 32) ss += row[j] * row[j];
  ss = rb_warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / (float)Dv + eps);
  for (int j = lane; j < Dv; j += 32) {
    const float g = rb_to_float<TI>(proj[(int64_t)t * ld + g_off + h * Dv + j]);
    const float gate = gate_silu ? g * sigmoidf_(g) : sigmoidf_(g);
    out[((int64_t)t * H + h) * Dv + j] = rb_from_float<TO>(row[j] * r * w[w_shared ? j : h * Dv + j] * gate);
  }
}

}  // namespace

RB_EXPORT int rb_conv_causal(float* u, const void* x, int64_t ldx, int x_off, int x_dtype, const float* x_bias,
                             const float* taps, const float* conv_bias, const float* tail, const int* tok_first,
                             const int* tok_slot, const int* tok_pos, int T, int C, int K, int silu, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(C > 0 && K >= 1, "rb_conv_causal: bad sizes C=%d K=%d", C, K);
  const int threads = 128;
  int by = (C + threads - 1) / threads;
  if (by > 64) by = 64;
  const int per_block = T >= 512 ? CONV_TOKENS : 1;
  const dim3 grid((T + per_block - 1) / per_block, by);
  if (x_dtype == RB_F32)
    RB_LAUNCH("conv_causal_kernel", (conv_causal_kernel<float>), grid, threads, 0, stream, u, (const float*)x, ldx, x_off, x_bias, taps, conv_bias, tail, tok_first, tok_slot, tok_pos, T, C, K, silu, per_block);
  else if (x_dtype == RB_BF16)
    RB_LAUNCH("conv_causal_kernel", (conv_causal_kernel<__nv_bfloat16>), grid, threads, 0, stream, u, (const __nv_bfloat16*)x, ldx, x_off, x_bias, taps, conv_bias, tail, tok_first, tok_slot, tok_pos, T, C, K, silu, per_block);
  else
    RB_FAIL("rb_conv_causal: unknown dtype %d", x_dtype);
  RB_CHECK_LAUNCH("rb_conv_causal");
  return 0;
}

// n_runs runs (seq_first, seq_count; null: every one of the n_runs rows is its own run).
RB_EXPORT int rb_conv_tail_update(float* tail, const void* x, int64_t ldx, int x_off, int x_dtype, const float* x_bias,
                                  const int* seq_first, const int* seq_count, const int* tok_slot, const int* tok_pos,
                                  int n_runs, int C, int K, cudaStream_t stream) {
  if (n_runs == 0 || K <= 1) return 0;
  RB_REQUIRE(C > 0, "rb_conv_tail_update: bad sizes C=%d", C);
  const int threads = 128;
  int by = (C + threads - 1) / threads;
  if (by > 64) by = 64;
  const dim3 grid(n_runs, by);
  if (x_dtype == RB_F32)
    RB_LAUNCH("conv_tail_kernel", (conv_tail_kernel<float>), grid, threads, 0, stream, tail, (const float*)x, ldx, x_off, x_bias, seq_first, seq_count, tok_slot, tok_pos, C, K);
  else if (x_dtype == RB_BF16)
    RB_LAUNCH("conv_tail_kernel", (conv_tail_kernel<__nv_bfloat16>), grid, threads, 0, stream, tail, (const __nv_bfloat16*)x, ldx, x_off, x_bias, seq_first, seq_count, tok_slot, tok_pos, C, K);
  else
    RB_FAIL("rb_conv_tail_update: unknown dtype %d", x_dtype);
  RB_CHECK_LAUNCH("rb_conv_tail_update");
  return 0;
}

// With seq_first and seq_count (runs of several rows; n_rows: all rows of the step) the gates buffer is overwritten.
RB_EXPORT int rb_gated_scan(void* out, int out_dtype, const float* u, const float* gates, const float* gate_r_bias,
                            const float* gate_i_bias, const float* lam, float decay_scale, const void* xy, int64_t ldxy,
                            int xy_dtype, int x_off, int y_off, const float* x_bias, const float* y_bias, float* state,
                            float* tail, const int* seq_first, const int* seq_count, const int* tok_slot, const int* tok_pos, int n_seq,
                            int n_rows, int W, int Wb, int K, cudaStream_t stream) {
  if (n_seq == 0) return 0;
  RB_REQUIRE(W > 0 && Wb > 0 && W % Wb == 0, "rb_gated_scan: width %d is not made of blocks of %d", W, Wb);
  RB_REQUIRE(K >= 1, "rb_gated_scan: %d taps", K);
  if (seq_first != nullptr && seq_count != nullptr) {
    // runs of several rows (a prompt, or a portion of one): decays and drives for all rows at once, then the chunked scan
    RB_REQUIRE(n_rows > 0, "rb_gated_scan: runs of several rows need the number of rows");
    const int64_t n = (int64_t)n_rows * W;
    const int64_t most = (int64_t)rb_sm_count() * 16;
    const int blocks = (int)((n + 255) / 256 < most ? (n + 255) / 256 : most);
    RB_LAUNCH("gate_prepare_kernel", (gate_prepare_kernel), blocks, 256, 0, stream, (float*)gates, u, gate_r_bias, gate_i_bias,
              lam, decay_scale, n, W, Wb);
    const dim3 cgrid(n_seq, (W + SCAN_CH - 1) / SCAN_CH);
#define CLAUNCH(TI, TO)                                                                                              \
  RB_LAUNCH("gated_scan_chunked_kernel", (gated_scan_chunked_kernel<TI, TO>), cgrid, SCAN_CH * SCAN_CHUNKS, 0, stream, \
            (TO*)out, gates, (const TI*)xy, ldxy, x_off, y_off, x_bias, y_bias, state, tail, seq_first, seq_count,   \
            tok_slot, tok_pos, W, Wb, K)
    if (xy_dtype == RB_F32 && out_dtype == RB_F32) CLAUNCH(float, float);
    else if (xy_dtype == RB_F32 && out_dtype == RB_BF16) CLAUNCH(float, __nv_bfloat16);
    else if (xy_dtype == RB_BF16 && out_dtype == RB_BF16) CLAUNCH(__nv_bfloat16, __nv_bfloat16);
    else RB_FAIL("rb_gated_scan: unsupported dtypes %d -> %d", xy_dtype, out_dtype);
#undef CLAUNCH
    RB_CHECK_LAUNCH("rb_gated_scan");
    return 0;
  }
  const dim3 grid(n_seq, (W + 63) / 64);
#define LAUNCH(TI, TO)                                                                                              \
  RB_LAUNCH("gated_scan_kernel", (gated_scan_kernel<TI, TO>), grid, 64, 0, stream, (TO*)out, u, gates, gate_r_bias,  \
            gate_i_bias, lam, decay_scale, (const TI*)xy, ldxy, x_off, y_off, x_bias, y_bias, state, tail, seq_first, \
            seq_count, tok_slot, tok_pos, W, Wb, K)
  if (xy_dtype == RB_F32 && out_dtype == RB_F32) LAUNCH(float, float);
  else if (xy_dtype == RB_F32 && out_dtype == RB_BF16) LAUNCH(float, __nv_bfloat16);
  else if (xy_dtype == RB_BF16 && out_dtype == RB_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else RB_FAIL("rb_gated_scan: unsupported dtypes %d -> %d", xy_dtype, out_dtype);
#undef LAUNCH
  RB_CHECK_LAUNCH("rb_gated_scan");
  return 0;
}

// Rows of which each is its own sequence, at most rb_gated_step_max_rows(): everything from the projections' rows to
// S_t * gelu_tanh(y_t) in one launch.  w_gates: [blocks, 2 Wb, Wb] float32 (recurrence gate's rows, then the input gate's).
RB_EXPORT int rb_gated_step_max_rows() { return STEP_MAX_ROWS; }

RB_EXPORT int rb_gated_step(void* out, int out_dtype, const void* xy, int64_t ldxy, int xy_dtype, int x_off, int y_off,
                            const float* x_bias, const float* y_bias, const float* taps, const float* conv_bias,
                            const float* w_gates, const float* gate_r_bias, const float* gate_i_bias, const float* lam,
                            float decay_scale, float* state, float* tail, const int* tok_slot, const int* tok_pos, int T, int W,
                            int Wb, int K, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(T <= STEP_MAX_ROWS, "rb_gated_step: %d rows (at most %d)", T, STEP_MAX_ROWS);
  RB_REQUIRE(W > 0 && Wb > 0 && W % Wb == 0 && K >= 1, "rb_gated_step: bad sizes W=%d Wb=%d K=%d", W, Wb, K);
  const size_t smem = (size_t)T * Wb * sizeof(float);
  RB_REQUIRE(smem <= 200 * 1024, "rb_gated_step: blocks of %d channels do not fit shared memory", Wb);
  const dim3 grid(W / Wb, (Wb + STEP_CH - 1) / STEP_CH);
#define LAUNCH(TI, TO)                                                                                                \
  do {                                                                                                                \
    if (smem > 48 * 1024)                                                                                             \
      RB_CUDA(cudaFuncSetAttribute(gated_step_kernel<TI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    RB_LAUNCH("gated_step_kernel", (gated_step_kernel<TI, TO>), grid, 32 * STEP_CH, smem, stream, (TO*)out, (const TI*)xy, ldxy, \
              x_off, y_off, x_bias, y_bias, taps, conv_bias, w_gates, gate_r_bias, gate_i_bias, lam, decay_scale, state, \
              tail, tok_slot, tok_pos, T, W, Wb, K);                                                                  \
  } while (0)
  if (xy_dtype == RB_F32 && out_dtype == RB_F32) LAUNCH(float, float);
  else if (xy_dtype == RB_F32 && out_dtype == RB_BF16) LAUNCH(float, __nv_bfloat16);
  else if (xy_dtype == RB_BF16 && out_dtype == RB_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else RB_FAIL("rb_gated_step: unsupported dtypes %d -> %d", xy_dtype, out_dtype);
#undef LAUNCH
  RB_CHECK_LAUNCH("rb_gated_step");
  return 0;
}

// Lanes per value column for a memory of D rows: the smallest power of two that leaves a thread at most 8 rows
// (16 rows beyond 256, where a warp's 32 lanes are all a column has).
RB_EXPORT int rb_matrix_memory_lanes(int D) {
  const int rows = D <= 128 ? 8 : 16;       // larger memories: 16 rows a thread, so that a block's copies of k and q serve more columns
  int P = 1;
  while ((D + P - 1) / P > rows && P < 32) P *= 2;
  return P;
}

template <int P, int R>
static int launch_matrix_memory(float* o_out, const float* proj, int64_t ld, int q_off, int k_off, int v_off, int i_off,
                                int f_off, const float* i_bias, const float* f_bias, float cap, float q_scale,
                                float floor_add, float* C_state, float* n_state, float* m_state, const int* seq_first,
                                const int* seq_count, const int* tok_slot, int n_seq, int H, int D, int Dv,
                                cudaStream_t stream) {
  // fewer columns per block while the blocks are too few to give every SM several: the work of a token is a
  // chain of dependent steps, and an SM hides it only behind other blocks' warps
  int threads = 128;
  const int64_t want = 3 * (int64_t)rb_sm_count();
  while (threads > 32 && threads / 2 >= P && (int64_t)n_seq * H * ((Dv + threads / P - 1) / (threads / P)) < want) threads /= 2;
  const int cols = threads / P;
  const int cols4 = (cols + 3) & ~3;
  const dim3 grid(n_seq, H, (Dv + cols - 1) / cols);
  RB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "rb_matrix_memory: grid %d x %d", grid.y, grid.z);
  const size_t smem = (size_t)(2 * MM_TT * (2 * P * R + cols4 + 4) + 3 * MM_TT + 4) * sizeof(float);
  const int vec4 = (D % 4 == 0 && ld % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && (uintptr_t)proj % 16 == 0) ? 1 : 0;
  static RbOncePerDevice once;
  if (smem > 48 * 1024 && once.first())
    RB_CUDA(cudaFuncSetAttribute(matrix_memory_kernel<P, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
  RB_LAUNCH("matrix_memory_kernel", (matrix_memory_kernel<P, R>), grid, threads, smem, stream, o_out, proj, ld, q_off, k_off,
            v_off, i_off, f_off, i_bias, f_bias, cap, q_scale, floor_add, C_state, n_state, m_state, seq_first, seq_count,
            tok_slot, H, D, Dv, vec4);
  RB_CHECK_LAUNCH("rb_matrix_memory");
  return 0;
}

RB_EXPORT int rb_matrix_memory(float* o_out, const void* proj, int64_t ld, int proj_dtype, int q_off, int k_off, int v_off,
                               int i_off, int f_off, const float* i_bias, const float* f_bias, float cap, float q_scale,
                               float floor_add, float* C_state, float* n_state, float* m_state, const int* seq_first,
                               const int* seq_count, const int* tok_slot, int n_seq, int H, int D, int Dv,
                               cudaStream_t stream) {
  if (n_seq == 0) return 0;
  RB_REQUIRE(H > 0 && D > 0 && Dv > 0 && D <= 512, "rb_matrix_memory: bad sizes H=%d D=%d Dv=%d (D up to 512)", H, D, Dv);
  RB_REQUIRE(cap > 0.f, "rb_matrix_memory: the gates' cap must be positive");
  RB_REQUIRE(proj_dtype == RB_F32, "rb_matrix_memory: the projections are float32 rows (found dtype %d)", proj_dtype);
  const int P = rb_matrix_memory_lanes(D);
  const int per = (D + P - 1) / P;
#define GO(PP, RR)                                                                                                    \
  return launch_matrix_memory<PP, RR>(o_out, (const float*)proj, ld, q_off, k_off, v_off, i_off, f_off, i_bias, f_bias, \
                                      cap, q_scale, floor_add, C_state, n_state, m_state, seq_first, seq_count,       \
                                      tok_slot, n_seq, H, D, Dv, stream)
  switch (P) {
    case 1: GO(1, 8);
    case 2: GO(2, 8);
    case 4: GO(4, 8);
    case 8: GO(8, 8);
    case 16:
      if (per <= 8) GO(16, 8);
      GO(16, 16);
    default:
      if (per <= 8) GO(32, 8);
      GO(32, 16);
  }
#undef GO
}

RB_EXPORT int rb_head_norm_gate(void* out, int out_dtype, const float* o, const float* w, const void* proj, int64_t ld,
                                int proj_dtype, int g_off, int T, int H, int Dv, float eps, int w_shared, int gate_silu,
                                cudaStream_t stream) {
  if (T == 0) return 0;
  const int64_t items = (int64_t)T * H;
  const int blocks = (int)((items + 3) / 4);
#define LAUNCH(TI, TO)                                                                                              \
  RB_LAUNCH("head_norm_gate_kernel", (head_norm_gate_kernel<TI, TO>), blocks, 128, 0, stream, (TO*)out, o, w,        \
            (const TI*)proj, ld, g_off, T, H, Dv, eps, w_shared, gate_silu)
  if (proj_dtype == RB_F32 && out_dtype == RB_F32) LAUNCH(float, float);
  else if (proj_dtype == RB_F32 && out_dtype == RB_BF16) LAUNCH(float, __nv_bfloat16);
  else if (proj_dtype == RB_BF16 && out_dtype == RB_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else RB_FAIL("rb_head_norm_gate: unsupported dtypes %d -> %d", proj_dtype, out_dtype);
#undef LAUNCH
  RB_CHECK_LAUNCH("rb_head_norm_gate");
  return 0;
}
