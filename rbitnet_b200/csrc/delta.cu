// The gated delta rule: a matrix memory per head that forgets by a decay and corrects what it holds for a key.
//
//   q, k: unit vectors per key head (x / sqrt(sum x^2 + unit_eps)), q also times q_scale
//   beta = sigmoid(b),  g = exp(-exp(A_log) * softplus(a + dt_bias))
//   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q          (S: [D, Dv] per head, float32)
//
// Value head h reads key head h / (H / G).  The read-out sees the token's own write: with r = S_old^T k and
// p = S_old^T q taken from the memory as the token found it, u = beta (v - g r) and o = g p + u (k . q), so that
// one pass over the memory serves both sums and the update S = g S_old + k u^T.
//
// A step brings, per sequence, a run of consecutive rows; the memory of the run's slot is read at its start and
// written back at its end (kept by value column: [slot, H, Dv, D]), so a prompt may arrive whole, in portions or
// token by token.  Everything here is float32.
#include "rb_common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

// ---------------------------------------------------------------- per token: unit vectors and gates
// u: rows [T, 2 G D + H Dv] (q heads, k heads, v heads) after the convolution and its activation; q and k are
// normalised in place.  proj: the projections' float32 rows with b at column b_off and a at column a_off.
// Leaves beta, decay [T, H] and kq [T, G] (the product k . q of the finished vectors).
__global__ void __launch_bounds__(128) delta_prepare_kernel(float* __restrict__ u, int64_t ldu, const float* __restrict__ proj,
                                                            int64_t ld, int b_off, int a_off, const float* __restrict__ A_log,
                                                            const float* __restrict__ dt_bias, float* __restrict__ beta,
                                                            float* __restrict__ decay, float* __restrict__ kq, int H, int G,
                                                            int D, float q_scale, float unit_eps) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  float* row = u + (int64_t)t * ldu;
  for (int g = warp; g < G; g += n_warps) {
    float* q = row + g * D;
    float* k = row + (G + g) * D;
    float sq = 0.f, sk = 0.f;
    for (int d = lane; d < D; d += 32) { sq = fmaf(q[d], q[d], sq); sk = fmaf(k[d], k[d], sk); }
    sq = rb_warp_sum(sq);
    sk = rb_warp_sum(sk);
    const float rq = q_scale / sqrtf(sq + unit_eps), rk = 1.0f / sqrtf(sk + unit_eps);
    float dot = 0.f;
    for (int d = lane; d < D; d += 32) {
      const float a = q[d] * rq, b = k[d] * rk;
      q[d] = a;
      k[d] = b;
      dot = fmaf(a, b, dot);
    }
    dot = rb_warp_sum(dot);
    if (lane == 0) kq[(int64_t)t * G + g] = dot;
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float* p = proj + (int64_t)t * ld;
    beta[(int64_t)t * H + h] = sigmoid_(p[b_off + h]);
    decay[(int64_t)t * H + h] = expf(-expf(A_log[h]) * softplus_(p[a_off + h] + dt_bias[h]));
  }
}

// ---------------------------------------------------------------- the recurrence
// A block per (run, head, tile of value columns).  A value column belongs to P neighbouring lanes (P a power of two
// up to 32); lane p of them holds rows d = p + P r (r < R) of the column in registers.  The run's tokens come through
// shared memory TT at a time: the head's k and q, the tile's values, the token's three numbers.
template <int R>
__global__ void __launch_bounds__(128) gated_delta_kernel(
    float* __restrict__ o, const float* __restrict__ u, int64_t ldu, const float* __restrict__ beta,
    const float* __restrict__ decay, const float* __restrict__ kq, float* __restrict__ state,
    const int* __restrict__ seq_first, const int* __restrict__ seq_count, const int* __restrict__ tok_slot, int H, int G,
    int D, int Dv, int P, int TT) {
  rb_pdl_launch_dependents();
  extern __shared__ float s_delta[];
  float* ks = s_delta;                    // [TT][D]
  float* qs = ks + (size_t)TT * D;        // [TT][D]
  const int CT = 128 / P;                 // value columns of this block
  float* vs = qs + (size_t)TT * D;        // [TT][CT]
  float* sc = vs + (size_t)TT * CT;       // [TT][3]: beta, decay, k . q
  const int h = blockIdx.y, kvh = h / (H / G);
  const int p = threadIdx.x % P, col = blockIdx.z * CT + threadIdx.x / P;
  const bool live = col < Dv;
  rb_pdl_wait();
  const int first = seq_first != nullptr ? seq_first[blockIdx.x] : blockIdx.x;
  const int n = seq_count != nullptr ? seq_count[blockIdx.x] : 1;
  const int slot = tok_slot[first];
  float* mine = state + (((int64_t)slot * H + h) * Dv + (live ? col : 0)) * D;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = p + P * r;
    S[r] = live && d < D ? mine[d] : 0.f;
  }
  const int q_off = kvh * D, k_off = (G + kvh) * D, v_off = 2 * G * D + h * Dv + blockIdx.z * CT;
  for (int c0 = 0; c0 < n; c0 += TT) {
    const int m = min(TT, n - c0);
    __syncthreads();
    for (int i = threadIdx.x; i < m * D; i += 128) {
      const int j = i / D, d = i - j * D;
      const float* row = u + (int64_t)(first + c0 + j) * ldu;
      ks[j * D + d] = row[k_off + d];
      qs[j * D + d] = row[q_off + d];
    }
    for (int i = threadIdx.x; i < m * CT; i += 128) {
      const int j = i / CT, c = i - j * CT;
      vs[j * CT + c] = blockIdx.z * CT + c < Dv ? u[(int64_t)(first + c0 + j) * ldu + v_off + c] : 0.f;
    }
    for (int j = threadIdx.x; j < m; j += 128) {
      const int64_t t = first + c0 + j;
      sc[j * 3 + 0] = beta[t * H + h];
      sc[j * 3 + 1] = decay[t * H + h];
      sc[j * 3 + 2] = kq[t * G + kvh];
    }
    __syncthreads();
    for (int j = 0; j < m; ++j) {
      const float* kj = ks + j * D;
      const float* qj = qs + j * D;
      float kr[R];
      float rsum = 0.f, psum = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int d = p + P * r;
        kr[r] = d < D ? kj[d] : 0.f;
        const float qd = d < D ? qj[d] : 0.f;
        rsum = fmaf(S[r], kr[r], rsum);
        psum = fmaf(S[r], qd, psum);
      }
      for (int off = P >> 1; off > 0; off >>= 1) {
        rsum += __shfl_xor_sync(0xffffffffu, rsum, off);
        psum += __shfl_xor_sync(0xffffffffu, psum, off);
      }
      const float b = sc[j * 3], g = sc[j * 3 + 1], dot = sc[j * 3 + 2];
      const float w = b * (vs[j * CT + threadIdx.x / P] - g * rsum);
#pragma unroll
      for (int r = 0; r < R; ++r) S[r] = fmaf(kr[r], w, g * S[r]);
      if (live && p == 0) o[((int64_t)(first + c0 + j) * H + h) * Dv + col] = fmaf(w, dot, g * psum);
    }
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = p + P * r;
      if (d < D) mine[d] = S[r];
    }
  }
}

}  // namespace

RB_EXPORT int rb_delta_prepare(float* u, int64_t ldu, const float* proj, int64_t ld, int b_off, int a_off, const float* A_log,
                               const float* dt_bias, float* beta, float* decay, float* kq, int T, int H, int G, int D,
                               float q_scale, float unit_eps, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(H > 0 && G > 0 && H % G == 0 && D > 0, "rb_delta_prepare: bad sizes H=%d G=%d D=%d", H, G, D);
  RB_LAUNCH("delta_prepare_kernel", (delta_prepare_kernel), T, 128, 0, stream, u, ldu, proj, ld, b_off, a_off, A_log, dt_bias,
            beta, decay, kq, H, G, D, q_scale, unit_eps);
  RB_CHECK_LAUNCH("rb_delta_prepare");
  return 0;
}

// o: [rows, H, Dv] float32.  u: rows [q heads (G D) | k heads (G D) | v heads (H Dv)], prepared.  state: [slots, H, Dv, D].
// n_runs runs (seq_first, seq_count; null: every one of the n_runs rows is its own run).
RB_EXPORT int rb_gated_delta(float* o, const float* u, int64_t ldu, const float* beta, const float* decay, const float* kq,
                             float* state, const int* seq_first, const int* seq_count, const int* tok_slot, int n_runs, int H,
                             int G, int D, int Dv, cudaStream_t stream) {
  if (n_runs == 0) return 0;
  RB_REQUIRE(H > 0 && G > 0 && H % G == 0 && D > 0 && Dv > 0 && D <= 1024, "rb_gated_delta: bad sizes H=%d G=%d D=%d Dv=%d", H, G, D, Dv);
  int P = 1;
  while (P < 32 && (D + P - 1) / P > 16) P *= 2;
  const int per = (D + P - 1) / P;
  const int CT = 128 / P;
  int TT = 16;
  while (TT > 1 && (size_t)TT * (2 * D + CT + 3) * sizeof(float) > 40 * 1024) TT /= 2;
  const size_t smem = (size_t)TT * (2 * D + CT + 3) * sizeof(float);
  const dim3 grid(n_runs, H, (Dv + CT - 1) / CT);
  RB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "rb_gated_delta: too many heads or columns");
  if (per <= 16)
    RB_LAUNCH("gated_delta_kernel", (gated_delta_kernel<16>), grid, 128, smem, stream, o, u, ldu, beta, decay, kq, state, seq_first,
              seq_count, tok_slot, H, G, D, Dv, P, TT);
  else
    RB_LAUNCH("gated_delta_kernel", (gated_delta_kernel<32>), grid, 128, smem, stream, o, u, ldu, beta, decay, kq, state, seq_first,
              seq_count, tok_slot, H, G, D, Dv, P, TT);
  RB_CHECK_LAUNCH("rb_gated_delta");
  return 0;
}
