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
// up to 32); lane p of them holds rows d = p R + r (r < R) of the column in registers.  The run's tokens come through
// shared memory TT at a time, copied a chunk ahead with cp.async into the other of two buffers: the head's k and q
// (each lane's R values followed by four floats of padding, so that the lanes' 16-byte loads fall into different
// banks), the tile's values, the token's three numbers.  Rows beyond D stay zero in both buffers.
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int P, int R, int NT>
__global__ void __launch_bounds__(NT) gated_delta_kernel(
    float* __restrict__ o, const float* __restrict__ u, int64_t ldu, const float* __restrict__ beta,
    const float* __restrict__ decay, const float* __restrict__ kq, float* __restrict__ state,
    const int* __restrict__ seq_first, const int* __restrict__ seq_count, const int* __restrict__ tok_slot, int H, int G,
    int D, int Dv, int TT, int vec16) {
  rb_pdl_launch_dependents();
  constexpr int CT = NT / P;              // value columns of this block
  constexpr int KS = P * (R + 4);         // floats of one token's k (or q) in shared memory
  extern __shared__ __align__(16) float s_delta[];
  constexpr int per_tok = 2 * KS + ((CT + 3) & ~3) + 4;      // a multiple of four floats: every token's k and q start on 16 bytes
  const int h = blockIdx.y, kvh = h / (H / G);
  const int p = threadIdx.x % P, cl = threadIdx.x / P, col = blockIdx.z * CT + cl;
  const bool live = col < Dv;
  for (int i = threadIdx.x; i < 2 * TT * per_tok; i += NT) s_delta[i] = 0.f;
  rb_pdl_wait();
  const int first = seq_first != nullptr ? seq_first[blockIdx.x] : blockIdx.x;
  const int n = seq_count != nullptr ? seq_count[blockIdx.x] : 1;
  const int slot = tok_slot[first];
  float* mine = state + (((int64_t)slot * H + h) * Dv + (live ? col : 0)) * D;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = p * R + r;
    S[r] = live && d < D ? mine[d] : 0.f;
  }
  const int q_off = kvh * D, k_off = (G + kvh) * D, v_off = 2 * G * D + h * Dv + blockIdx.z * CT;
  __syncthreads();                        // the buffers are zero before the first copies land
  auto copy_chunk = [&](int c0, int buf) {
    const int m = min(TT, n - c0);
    float* base = s_delta + (size_t)buf * TT * per_tok;
    if (vec16) {
      const int D4 = D >> 2;
      for (int i = threadIdx.x; i < m * D4; i += NT) {
        const int j = i / D4, d = (i - j * D4) << 2;
        const float* row = u + (int64_t)(first + c0 + j) * ldu;
        float* dst = base + (size_t)j * per_tok + (d / R) * (R + 4) + d % R;
        cp_async16(dst, row + k_off + d);
        cp_async16(dst + KS, row + q_off + d);
      }
    } else {
      for (int i = threadIdx.x; i < m * D; i += NT) {
        const int j = i / D, d = i - j * D;
        const float* row = u + (int64_t)(first + c0 + j) * ldu;
        float* dst = base + (size_t)j * per_tok + (d / R) * (R + 4) + d % R;
        cp_async4(dst, row + k_off + d);
        cp_async4(dst + KS, row + q_off + d);
      }
    }
    for (int i = threadIdx.x; i < m * CT; i += NT) {
      const int j = i / CT, c = i - j * CT;
      if (blockIdx.z * CT + c < Dv) cp_async4(base + (size_t)j * per_tok + 2 * KS + c, u + (int64_t)(first + c0 + j) * ldu + v_off + c);
    }
    for (int j = threadIdx.x; j < m; j += NT) {
      const int64_t t = first + c0 + j;
      float* dst = base + (size_t)j * per_tok + 2 * KS + ((CT + 3) & ~3);
      cp_async4(dst, beta + t * H + h);
      cp_async4(dst + 1, decay + t * H + h);
      cp_async4(dst + 2, kq + t * G + kvh);
    }
  };
  copy_chunk(0, 0);
  cp_async_commit();
  int buf = 0;
  for (int c0 = 0; c0 < n; c0 += TT, buf ^= 1) {
    const int m = min(TT, n - c0);
    if (c0 + TT < n) {
      copy_chunk(c0 + TT, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* base = s_delta + (size_t)buf * TT * per_tok;
    for (int j = 0; j < m; ++j) {
      const float* tok = base + (size_t)j * per_tok;
      const float4* k4 = reinterpret_cast<const float4*>(tok + p * (R + 4));
      const float4* q4 = reinterpret_cast<const float4*>(tok + KS + p * (R + 4));
      float kr[R];
      float rs[4] = {0.f, 0.f, 0.f, 0.f}, ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < R / 4; ++i) {
        const float4 kk = k4[i], qq = q4[i];
        kr[4 * i] = kk.x; kr[4 * i + 1] = kk.y; kr[4 * i + 2] = kk.z; kr[4 * i + 3] = kk.w;
        rs[0] = fmaf(S[4 * i], kk.x, rs[0]); rs[1] = fmaf(S[4 * i + 1], kk.y, rs[1]);
        rs[2] = fmaf(S[4 * i + 2], kk.z, rs[2]); rs[3] = fmaf(S[4 * i + 3], kk.w, rs[3]);
        ps[0] = fmaf(S[4 * i], qq.x, ps[0]); ps[1] = fmaf(S[4 * i + 1], qq.y, ps[1]);
        ps[2] = fmaf(S[4 * i + 2], qq.z, ps[2]); ps[3] = fmaf(S[4 * i + 3], qq.w, ps[3]);
      }
      float rsum = (rs[0] + rs[1]) + (rs[2] + rs[3]), psum = (ps[0] + ps[1]) + (ps[2] + ps[3]);
#pragma unroll
      for (int off = P >> 1; off > 0; off >>= 1) {
        rsum += __shfl_xor_sync(0xffffffffu, rsum, off);
        psum += __shfl_xor_sync(0xffffffffu, psum, off);
      }
      const float* sc = tok + 2 * KS + ((CT + 3) & ~3);
      const float b = sc[0], g = sc[1], dot = sc[2];
      const float w = b * (tok[2 * KS + cl] - g * rsum);
#pragma unroll
      for (int r = 0; r < R; ++r) S[r] = fmaf(kr[r], w, g * S[r]);
      if (live && p == 0) o[((int64_t)(first + c0 + j) * H + h) * Dv + col] = fmaf(w, dot, g * psum);
    }
    __syncthreads();                      // before the copies of the chunk after the next overwrite this buffer
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = p * R + r;
      if (d < D) mine[d] = S[r];
    }
  }
}

template <int P, int R, int NT>
int launch_delta(dim3 grid, size_t smem, cudaStream_t stream, float* o, const float* u, int64_t ldu, const float* beta,
                 const float* decay, const float* kq, float* state, const int* seq_first, const int* seq_count,
                 const int* tok_slot, int H, int G, int D, int Dv, int TT, int vec16) {
  RB_LAUNCH("gated_delta_kernel", (gated_delta_kernel<P, R, NT>), grid, NT, smem, stream, o, u, ldu, beta, decay, kq, state,
            seq_first, seq_count, tok_slot, H, G, D, Dv, TT, vec16);
  RB_CHECK_LAUNCH("rb_gated_delta");
  return 0;
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
  const int R = (D + P - 1) / P > 16 ? 32 : 16;
  // blocks of 64 threads where blocks of 128 would leave SMs without one
  const long long blocks128 = (long long)n_runs * H * ((Dv + 128 / P - 1) / (128 / P));
  const int NT = blocks128 < 2ll * rb_sm_count() ? 64 : 128;
  const int CT = NT / P;
  const int per_tok = 2 * P * (R + 4) + ((CT + 3) & ~3) + 4;
  int TT = 16;
  while (TT > 1 && (size_t)2 * TT * per_tok * sizeof(float) > 46 * 1024) TT /= 2;
  const size_t smem = (size_t)2 * TT * per_tok * sizeof(float);
  RB_REQUIRE(smem <= 48 * 1024, "rb_gated_delta: key size %d needs %zu bytes of shared memory", D, smem);
  const dim3 grid(n_runs, H, (Dv + CT - 1) / CT);
  RB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "rb_gated_delta: too many heads or columns");
  const int vec16 = D % 4 == 0 && ldu % 4 == 0 && (uintptr_t)u % 16 == 0 && (G * D) % 4 == 0;
#define GO(PP, RR)                                                                                                          \
  if (P == PP && R == RR)                                                                                                   \
    return NT == 64 ? launch_delta<PP, RR, 64>(grid, smem, stream, o, u, ldu, beta, decay, kq, state, seq_first, seq_count, \
                                               tok_slot, H, G, D, Dv, TT, vec16)                                            \
                    : launch_delta<PP, RR, 128>(grid, smem, stream, o, u, ldu, beta, decay, kq, state, seq_first, seq_count, \
                                                tok_slot, H, G, D, Dv, TT, vec16)
  GO(1, 16); GO(2, 16); GO(4, 16); GO(8, 16); GO(16, 16); GO(32, 16); GO(32, 32);
#undef GO
  RB_FAIL("rb_gated_delta: no kernel for a key size of %d", D);
}
