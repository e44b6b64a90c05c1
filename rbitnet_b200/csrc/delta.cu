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
// Leaves beta, decay and its logarithm [T, H], and kq [T, G] (the product k . q of the finished vectors).
__global__ void __launch_bounds__(128) delta_prepare_kernel(float* __restrict__ u, int64_t ldu, const float* __restrict__ proj,
                                                            int64_t ld, int b_off, int a_off, const float* __restrict__ A_log,
                                                            const float* __restrict__ dt_bias, float* __restrict__ beta,
                                                            float* __restrict__ decay, float* __restrict__ log_decay,
                                                            float* __restrict__ kq, int H, int G, int D, float q_scale,
                                                            float unit_eps) {
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
    const float lg = -expf(A_log[h]) * softplus_(p[a_off + h] + dt_bias[h]);
    decay[(int64_t)t * H + h] = expf(lg);
    log_decay[(int64_t)t * H + h] = lg;
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
  if (D != P * R)                         // rows beyond D are read as zeros
    for (int i = threadIdx.x; i < 2 * TT * per_tok; i += NT) s_delta[i] = 0.f;
  rb_pdl_wait();
  const int first = seq_first != nullptr ? seq_first[blockIdx.x] : blockIdx.x;
  const int n = seq_count != nullptr ? seq_count[blockIdx.x] : 1;
  const int slot = tok_slot[first];
  float* mine = state + (((int64_t)slot * H + h) * Dv + (live ? col : 0)) * D;
  float S[R];
  if (D == P * R) {
    // whole rows: 16 bytes at a time (D is a multiple of 16 here, and a column's rows start on 16 bytes)
#pragma unroll
    for (int r = 0; r < R; r += 4) {
      const float4 f = live ? *reinterpret_cast<const float4*>(mine + p * R + r) : make_float4(0.f, 0.f, 0.f, 0.f);
      S[r] = f.x; S[r + 1] = f.y; S[r + 2] = f.z; S[r + 3] = f.w;
    }
  } else {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = p * R + r;
      S[r] = live && d < D ? mine[d] : 0.f;
    }
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
  if (live && D == P * R) {
#pragma unroll
    for (int r = 0; r < R; r += 4) *reinterpret_cast<float4*>(mine + p * R + r) = make_float4(S[r], S[r + 1], S[r + 2], S[r + 3]);
  } else if (live) {
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

// ---------------------------------------------------------------- a decode step in one launch
// One token per sequence: a block per (row, head) does everything between the stacked product and the output product:
// the convolution of the head's q, k and v channels from the ring of last inputs (and the ring's new row), SiLU, the
// unit vectors, beta and the decay, one step of the memory for all of the head's value columns (a column on P lanes of
// R rows each), the norm over the head's outputs, the weight and the SiLU gate.  q and k of a key head are made again by
// every value head that reads it; the first of them writes their ring rows.
template <int R>
__global__ void __launch_bounds__(1024) delta_step_kernel(
    void* __restrict__ out, int out_bf16, const float* __restrict__ proj, int64_t ld, int g_off, int b_off, int a_off,
    const float* __restrict__ taps, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
    const float* __restrict__ norm_w, float* __restrict__ state, float* __restrict__ tail, const int* __restrict__ tok_slot,
    const int* __restrict__ tok_pos, int H, int G, int D, int Dv, int K, int P, float q_scale, float unit_eps, float norm_eps) {
  rb_pdl_launch_dependents();
  extern __shared__ __align__(16) float s_step[];
  __shared__ float scratch[33];
  float* qs = s_step;            // [D]
  float* ks = qs + D;            // [D]
  float* vs = ks + D;            // [Dv]
  const int t = blockIdx.x, h = blockIdx.y, kvh = h / (H / G), tid = threadIdx.x;
  const int C = 2 * G * D + H * Dv;
  rb_pdl_wait();
  const int slot = tok_slot[t], pos = tok_pos[t];
  const float* row = proj + (int64_t)t * ld;
  const bool writes_qk = h % (H / G) == 0;
  for (int i = tid; i < 2 * D + Dv; i += blockDim.x) {
    const int ch = i < D ? kvh * D + i : (i < 2 * D ? (G + kvh) * D + (i - D) : 2 * G * D + h * Dv + (i - 2 * D));
    const float x0 = row[ch];
    float acc = taps[(int64_t)ch * K + (K - 1)] * x0;
    for (int d = 1; d < K; ++d) {
      if (pos - d < 0) break;
      acc = fmaf(taps[(int64_t)ch * K + (K - 1 - d)], tail[((int64_t)slot * K + (pos - d) % K) * C + ch], acc);
    }
    if (K > 1 && (i >= 2 * D || writes_qk)) tail[((int64_t)slot * K + pos % K) * C + ch] = x0;
    s_step[i] = acc * sigmoid_(acc);
  }
  __syncthreads();
  float sq = 0.f, sk = 0.f;
  for (int d = tid; d < D; d += blockDim.x) { sq = fmaf(qs[d], qs[d], sq); sk = fmaf(ks[d], ks[d], sk); }
  sq = rb_block_sum(sq, scratch);
  sk = rb_block_sum(sk, scratch);
  const float rq = q_scale / sqrtf(sq + unit_eps), rk = 1.0f / sqrtf(sk + unit_eps);
  float dot = 0.f;
  for (int d = tid; d < D; d += blockDim.x) {
    const float a = qs[d] * rq, b = ks[d] * rk;
    qs[d] = a;
    ks[d] = b;
    dot = fmaf(a, b, dot);
  }
  dot = rb_block_sum(dot, scratch);          // (its barriers also make the finished q and k visible)
  const float beta = sigmoid_(row[b_off + h]);
  const float g = expf(-expf(A_log[h]) * softplus_(row[a_off + h] + dt_bias[h]));
  const int p = tid % P, col = tid / P;
  const bool live = col < Dv;
  float o = 0.f;
  {
    // every thread walks this part, also those beyond the head's columns (with zeros): the lanes of a warp meet in the
    // shuffles below
    float* mine = state + (((int64_t)slot * H + h) * Dv + (live ? col : 0)) * D;
    float S[R];
    float rsum = 0.f, psum = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = p * R + r;
      const bool in = live && d < D;
      S[r] = in ? mine[d] : 0.f;
      rsum = fmaf(S[r], in ? ks[d] : 0.f, rsum);
      psum = fmaf(S[r], in ? qs[d] : 0.f, psum);
    }
    for (int off = P >> 1; off > 0; off >>= 1) {
      rsum += __shfl_xor_sync(0xffffffffu, rsum, off);
      psum += __shfl_xor_sync(0xffffffffu, psum, off);
    }
    if (live) {
      const float w = beta * (vs[col] - g * rsum);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int d = p * R + r;
        if (d < D) mine[d] = fmaf(ks[d], w, g * S[r]);
      }
      o = fmaf(w, dot, g * psum);
    }
  }
  const float ss = rb_block_sum(live && p == 0 ? o * o : 0.f, scratch);
  if (live && p == 0) {
    const float r = 1.0f / sqrtf(ss / (float)Dv + norm_eps);
    const float gate = row[g_off + h * Dv + col];
    const float y = o * r * norm_w[col] * (gate * sigmoid_(gate));
    const int64_t at = ((int64_t)t * H + h) * Dv + col;
    if (out_bf16) ((__nv_bfloat16*)out)[at] = __float2bfloat16_rn(y);
    else ((float*)out)[at] = y;
  }
}

// ---------------------------------------------------------------- long runs: chunks of 32 tokens
// Within a chunk that starts from the memory S0, with L_i the sum of the logarithms of the decays of the chunk's tokens
// up to i (so that exp(L_i - L_j) is the decay from token j to token i):
//   u_i = beta_i (v_i - e^{L_i} S0^T k_i - sum_{j<i} e^{L_i - L_j} (k_i . k_j) u_j)
// which is the triangular system (I + A) U = diag(beta) V - diag(beta e^L) K S0, A_ij = beta_i e^{L_i - L_j} (k_i . k_j), j < i.
// With T = (I + A)^-1:  Ut = T diag(beta) V,  W = T diag(beta e^L) K,  U = Ut - W S0, and then
//   o_i = e^{L_i} S0^T q_i + sum_{j<=i} M_ij u_j,  M_ij = e^{L_i - L_j} (q_i . k_j)
//   S_end = e^{L_end} S0 + sum_j e^{L_end - L_j} k_j u_j^T
// The first kernel makes W, Ut, M and L for every (chunk, head) at once; the second walks a run's chunks with the memory,
// three small products per chunk.  A chunk's missing tokens (the run's end) count as beta = 0, decay 1, k = q = v = 0.
constexpr int CH = 32;

// grid (chunks, H), 128 threads.  chunk_row[c]: the chunk's first row; chunk_len[c]: its tokens (1..32).
// Scratch per (chunk, head): W [32][D], Ut [32][Dv], M [32][32], L [32].
__global__ void __launch_bounds__(128) delta_chunk_prepare_kernel(
    float* __restrict__ Wg, float* __restrict__ Utg, float* __restrict__ Mg, float* __restrict__ Lg,
    const float* __restrict__ u, int64_t ldu, const float* __restrict__ beta, const float* __restrict__ log_decay,
    const int* __restrict__ chunk_row, const int* __restrict__ chunk_len, int H, int G, int D, int Dv) {
  rb_pdl_launch_dependents();
  extern __shared__ __align__(16) float s_prep[];
  const int KS = D + 4;                          // row stride of k and q
  float* Ks = s_prep;                            // [32][D + 4]
  float* Qs = Ks + CH * KS;                      // [32][D + 4]
  float* As = Qs + CH * KS;                      // [32][33]: the system's matrix below the diagonal
  float* Lc = As + CH * 33;                      // [32]
  float* Bt = Lc + CH;                           // [32]
  const int chunk = blockIdx.x, h = blockIdx.y, kvh = h / (H / G);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  rb_pdl_wait();
  const int row0 = chunk_row[chunk], m = chunk_len[chunk];
  const int q_off = kvh * D, k_off = (G + kvh) * D, v_off = 2 * G * D + h * Dv;
  for (int i = tid; i < CH * (D >> 2); i += 128) {
    const int j = i / (D >> 2), d = (i - j * (D >> 2)) << 2;
    float4 kk = make_float4(0.f, 0.f, 0.f, 0.f), qq = kk;
    if (j < m) {
      const float* row = u + (int64_t)(row0 + j) * ldu;
      kk = *reinterpret_cast<const float4*>(row + k_off + d);
      qq = *reinterpret_cast<const float4*>(row + q_off + d);
    }
    *reinterpret_cast<float4*>(Ks + j * KS + d) = kk;
    *reinterpret_cast<float4*>(Qs + j * KS + d) = qq;
  }
  if (warp == 0) {
    // the running sum of the logarithms, lane by lane
    float l = lane < m ? log_decay[(int64_t)(row0 + lane) * H + h] : 0.f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, l, o);
      if (lane >= o) l += up;
    }
    Lc[lane] = l;
    Bt[lane] = lane < m ? beta[(int64_t)(row0 + lane) * H + h] : 0.f;
  }
  __syncthreads();
  {
    // thread: column j = lane, rows i = warp + 4 r: the products k_i . k_j and q_i . k_j
    const int j = lane;
    float accA[8], accB[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) accA[r] = accB[r] = 0.f;
    for (int d = 0; d < D; d += 4) {
      const float4 kj = *reinterpret_cast<const float4*>(Ks + j * KS + d);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int i = warp + 4 * r;
        const float4 ki = *reinterpret_cast<const float4*>(Ks + i * KS + d);
        const float4 qi = *reinterpret_cast<const float4*>(Qs + i * KS + d);
        accA[r] = fmaf(ki.x, kj.x, fmaf(ki.y, kj.y, fmaf(ki.z, kj.z, fmaf(ki.w, kj.w, accA[r]))));
        accB[r] = fmaf(qi.x, kj.x, fmaf(qi.y, kj.y, fmaf(qi.z, kj.z, fmaf(qi.w, kj.w, accB[r]))));
      }
    }
    float* Mo = Mg + ((int64_t)chunk * H + h) * CH * CH;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int i = warp + 4 * r;
      const float f = j <= i ? expf(Lc[i] - Lc[j]) : 0.f;
      As[i * 33 + j] = j < i ? Bt[i] * f * accA[r] : 0.f;
      Mo[i * CH + j] = f * accB[r];
    }
    if (tid < CH) Lg[((int64_t)chunk * H + h) * CH + tid] = Lc[tid];
  }
  __syncthreads();
  // one column of the right-hand side per thread and turn: forward substitution down its 32 rows
  float* Wo = Wg + ((int64_t)chunk * H + h) * CH * D;
  float* Uo = Utg + ((int64_t)chunk * H + h) * CH * Dv;
  for (int c = tid; c < D + Dv; c += 128) {
    float X[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      float acc;
      if (c < D) acc = Bt[i] * expf(Lc[i]) * Ks[i * KS + c];
      else acc = i < m ? Bt[i] * u[(int64_t)(row0 + i) * ldu + v_off + (c - D)] : 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) acc = fmaf(-As[i * 33 + j], X[j], acc);
      X[i] = acc;
    }
    if (c < D) {
#pragma unroll
      for (int i = 0; i < CH; ++i) Wo[i * D + c] = X[i];
    } else {
#pragma unroll
      for (int i = 0; i < CH; ++i) Uo[i * Dv + (c - D)] = X[i];
    }
  }
}

// grid (runs, H, tiles of CT = 16 value columns), 256 threads (eight warps: two per scheduler, so that one's
// shared-memory loads run under the other's multiply-adds).  Shared memory: two buffers of a chunk's W, q, k
// [32][D] each, M [32][32] and L [32], filled a chunk ahead with cp.async; the memory's tile S [D][16], U [32][16] and
// the chunk's 2 x 32 exponentials.
constexpr int CCT = 16;
constexpr int SCAN_NT = 256;              // threads: 16 columns by SCAN_G groups of rows
constexpr int SCAN_G = SCAN_NT / CCT;      // 16
constexpr int SCAN_R = CH / SCAN_G;        // rows of a chunk per thread: 2
__device__ __forceinline__ void cp_async16_or_zeros(void* dst, const void* src, bool real) {
  const int bytes = real ? 16 : 0;            // fewer source bytes than 16: the rest is filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes)
               : "memory");
}

__global__ void __launch_bounds__(SCAN_NT) delta_chunk_scan_kernel(
    float* __restrict__ o, const float* __restrict__ Wg, const float* __restrict__ Utg, const float* __restrict__ Mg,
    const float* __restrict__ Lg, const float* __restrict__ u, int64_t ldu, float* __restrict__ state,
    const int* __restrict__ seq_first, const int* __restrict__ seq_count, const int* __restrict__ run_chunk0,
    const int* __restrict__ tok_slot, int H, int G, int D, int Dv) {
  rb_pdl_launch_dependents();
  extern __shared__ __align__(16) float s_scan[];
  const int per_buf = 3 * CH * D + CH * CH + CH;
  float* Ss = s_scan + 2 * per_buf;   // [D][16]
  float* Us = Ss + D * CCT;           // [32][16]
  float* Es = Us + CH * CCT;          // [32]: e^{L_i}
  float* Fs = Es + CH;                // [32]: e^{L_end - L_j}
  const int run = blockIdx.x, h = blockIdx.y, kvh = h / (H / G), col0 = blockIdx.z * CCT;
  const int tid = threadIdx.x, c = tid & 15, g8 = tid >> 4;          // column of the tile; one of SCAN_G groups of rows
  const bool live = col0 + c < Dv;
  rb_pdl_wait();
  const int first = seq_first[run], n = seq_count[run], chunk0 = run_chunk0[run];
  const int slot = tok_slot[first];
  const int q_off = kvh * D, k_off = (G + kvh) * D;
  const int D4 = D >> 2;
  auto copy_chunk = [&](int ci, int buf) {
    const int row0 = first + ci * CH, m = min(CH, n - ci * CH);
    const int64_t item = (int64_t)(chunk0 + ci) * H + h;
    float* Ws = s_scan + (size_t)buf * per_buf;
    float* Qs = Ws + CH * D;
    float* Kc = Qs + CH * D;
    float* Ms = Kc + CH * D;
    float* Ls = Ms + CH * CH;
    for (int i = tid; i < CH * D4; i += SCAN_NT) {
      const int j = i / D4, d = (i - j * D4) << 2;
      cp_async16(Ws + j * D + d, Wg + item * CH * D + j * D + d);
      const float* row = u + (int64_t)(row0 + (j < m ? j : 0)) * ldu;
      cp_async16_or_zeros(Kc + j * D + d, row + k_off + d, j < m);
      cp_async16_or_zeros(Qs + j * D + d, row + q_off + d, j < m);
    }
    for (int i = tid; i < CH * CH / 4; i += SCAN_NT) cp_async16(Ms + 4 * i, Mg + item * CH * CH + 4 * i);
    if (tid < CH / 4) cp_async16(Ls + 4 * tid, Lg + item * CH + 4 * tid);
  };
  const int n_chunks = (n + CH - 1) / CH;
  copy_chunk(0, 0);
  cp_async_commit();
  float* mine = state + (((int64_t)slot * H + h) * Dv + col0) * D;      // [column][D]
  for (int i = tid; i < D * CCT; i += SCAN_NT) {
    const int cc = i / D, d = i - cc * D;
    Ss[d * CCT + cc] = col0 + cc < Dv ? mine[(int64_t)cc * D + d] : 0.f;
  }
  for (int ci = 0, buf = 0; ci < n_chunks; ++ci, buf ^= 1) {
    const int row0 = first + ci * CH, m = min(CH, n - ci * CH);
    const int64_t item = (int64_t)(chunk0 + ci) * H + h;
    if (ci + 1 < n_chunks) {
      copy_chunk(ci + 1, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();                  // this chunk's copies have landed; S is in place
    const float* Ws = s_scan + (size_t)buf * per_buf;
    const float* Qs = Ws + CH * D;
    const float* Kc = Qs + CH * D;
    const float* Ms = Kc + CH * D;
    const float* Ls = Ms + CH * CH;
    // asked for now, used after the products
    const float* Ut = Utg + item * CH * Dv;
    float ut[SCAN_R];
#pragma unroll
    for (int r = 0; r < SCAN_R; ++r) ut[r] = live ? Ut[(int64_t)(g8 + SCAN_G * r) * Dv + col0 + c] : 0.f;
    if (tid < CH) {
      Es[tid] = expf(Ls[tid]);
      Fs[tid] = expf(Ls[CH - 1] - Ls[tid]);
    }
    // rows i = g8 + SCAN_G r (r < SCAN_R) of column c:  W S and Q S
    float ws[SCAN_R], qs[SCAN_R];
#pragma unroll
    for (int r = 0; r < SCAN_R; ++r) ws[r] = qs[r] = 0.f;
    for (int d = 0; d < D; d += 4) {
      const float s0 = Ss[d * CCT + c], s1 = Ss[(d + 1) * CCT + c], s2 = Ss[(d + 2) * CCT + c], s3 = Ss[(d + 3) * CCT + c];
#pragma unroll
      for (int r = 0; r < SCAN_R; ++r) {
        const int i = g8 + SCAN_G * r;
        const float4 w4 = *reinterpret_cast<const float4*>(Ws + i * D + d);
        const float4 q4 = *reinterpret_cast<const float4*>(Qs + i * D + d);
        ws[r] = fmaf(w4.x, s0, fmaf(w4.y, s1, fmaf(w4.z, s2, fmaf(w4.w, s3, ws[r]))));
        qs[r] = fmaf(q4.x, s0, fmaf(q4.y, s1, fmaf(q4.z, s2, fmaf(q4.w, s3, qs[r]))));
      }
    }
#pragma unroll
    for (int r = 0; r < SCAN_R; ++r) Us[(g8 + SCAN_G * r) * CCT + c] = ut[r] - ws[r];
    __syncthreads();
    // the chunk's outputs: e^{L_i} (Q S)_i + sum_{j <= i} M_ij U_j
#pragma unroll
    for (int r = 0; r < SCAN_R; ++r) {
      const int i = g8 + SCAN_G * r;
      float acc = Es[i] * qs[r];
      for (int j = 0; j <= i; ++j) acc = fmaf(Ms[i * CH + j], Us[j * CCT + c], acc);
      if (live && i < m) o[((int64_t)(row0 + i) * H + h) * Dv + col0 + c] = acc;
    }
    // the memory moves on: S <- e^{L_end} S + sum_j e^{L_end - L_j} k_j U_j, rows d = d0 + g8 + SCAN_G r of column c
    const float keep = Es[CH - 1];
    for (int d0 = 0; d0 < D; d0 += 8 * SCAN_G) {
      float acc[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) acc[r] = 0.f;
      for (int j = 0; j < CH; ++j) {
        const float uj = Fs[j] * Us[j * CCT + c];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const int d = d0 + g8 + SCAN_G * r;
          if (d < D) acc[r] = fmaf(Kc[j * D + d], uj, acc[r]);
        }
      }
      // (every thread read the old S in the products above, before the barrier that followed them)
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int d = d0 + g8 + SCAN_G * r;
        if (d < D) Ss[d * CCT + c] = fmaf(keep, Ss[d * CCT + c], acc[r]);
      }
    }
    __syncthreads();                  // before the copies of the chunk after the next overwrite this buffer, and U and the exponentials change
  }
  for (int i = tid; i < D * CCT; i += SCAN_NT) {
    const int cc = i / D, d = i - cc * D;
    if (col0 + cc < Dv) mine[(int64_t)cc * D + d] = Ss[d * CCT + cc];
  }
}

}  // namespace

RB_EXPORT int rb_delta_prepare(float* u, int64_t ldu, const float* proj, int64_t ld, int b_off, int a_off, const float* A_log,
                               const float* dt_bias, float* beta, float* decay, float* log_decay, float* kq, int T, int H,
                               int G, int D, float q_scale, float unit_eps, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(H > 0 && G > 0 && H % G == 0 && D > 0, "rb_delta_prepare: bad sizes H=%d G=%d D=%d", H, G, D);
  RB_LAUNCH("delta_prepare_kernel", (delta_prepare_kernel), T, 128, 0, stream, u, ldu, proj, ld, b_off, a_off, A_log, dt_bias,
            beta, decay, log_decay, kq, H, G, D, q_scale, unit_eps);
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
  int TT = seq_first == nullptr ? 1 : 16;         // every row its own run: one token a chunk
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

// Whether runs of several tokens take the chunked kernels (key sizes that are multiples of 4, up to 128, 16-byte rows).
RB_EXPORT int rb_gated_delta_chunked_supports(int D, int Dv, long long ldu, int G) {
  return D % 4 == 0 && D <= 128 && Dv > 0 && ldu % 4 == 0 && (G * D) % 4 == 0;
}

// Floats of scratch per (chunk, head): W, Ut, M, L.
RB_EXPORT long long rb_gated_delta_chunk_floats(int D, int Dv) { return (long long)CH * (D + Dv + CH + 1); }

// The same recurrence for runs of several tokens, in chunks of 32 (see above).  chunk_row, chunk_len: every chunk of
// every run, the runs' chunks in order; run_chunk0[r]: the first chunk of run r.  scratch: n_chunks * H *
// rb_gated_delta_chunk_floats(D, Dv) floats.
RB_EXPORT int rb_gated_delta_chunked(float* o, const float* u, int64_t ldu, const float* beta, const float* log_decay,
                                     float* state, float* scratch, const int* seq_first, const int* seq_count,
                                     const int* run_chunk0, const int* chunk_row, const int* chunk_len, const int* tok_slot,
                                     int n_runs, int n_chunks, int H, int G, int D, int Dv, cudaStream_t stream) {
  if (n_runs == 0 || n_chunks == 0) return 0;
  RB_REQUIRE(H > 0 && G > 0 && H % G == 0 && rb_gated_delta_chunked_supports(D, Dv, ldu, G) && (uintptr_t)u % 16 == 0 &&
                 (uintptr_t)scratch % 16 == 0,
             "rb_gated_delta_chunked: bad sizes H=%d G=%d D=%d Dv=%d", H, G, D, Dv);
  const int64_t items = (int64_t)n_chunks * H;
  float* Wg = scratch;
  float* Utg = Wg + items * CH * D;
  float* Mg = Utg + items * CH * Dv;
  float* Lg = Mg + items * CH * CH;
  RB_REQUIRE(n_chunks <= 2147483647 / 1 && H <= 65535, "rb_gated_delta_chunked: too many heads");
  const size_t smem_a = (size_t)(2 * CH * (D + 4) + CH * 33 + 2 * CH) * sizeof(float);
  const size_t smem_b = (size_t)(2 * (3 * CH * D + CH * CH + CH) + D * CCT + CH * CCT + 2 * CH) * sizeof(float);
  static RbOncePerDevice configured;
  if (configured.first()) {
    RB_CUDA(cudaFuncSetAttribute(delta_chunk_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
    RB_CUDA(cudaFuncSetAttribute(delta_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
  }
  RB_REQUIRE(smem_a <= 64 * 1024 && smem_b <= 128 * 1024, "rb_gated_delta_chunked: key size %d needs too much shared memory", D);
  RB_LAUNCH("delta_chunk_prepare_kernel", (delta_chunk_prepare_kernel), dim3(n_chunks, H), 128, smem_a, stream, Wg, Utg, Mg, Lg, u,
            ldu, beta, log_decay, chunk_row, chunk_len, H, G, D, Dv);
  RB_CHECK_LAUNCH("rb_gated_delta_chunked");
  const dim3 grid(n_runs, H, (Dv + CCT - 1) / CCT);
  RB_REQUIRE(grid.z <= 65535, "rb_gated_delta_chunked: too many columns");
  RB_LAUNCH("delta_chunk_scan_kernel", (delta_chunk_scan_kernel), grid, SCAN_NT, smem_b, stream, o, Wg, Utg, Mg, Lg, u, ldu, state,
            seq_first, seq_count, run_chunk0, tok_slot, H, G, D, Dv);
  RB_CHECK_LAUNCH("rb_gated_delta_chunked");
  return 0;
}

// Lanes per value column of the one-launch decode step for these sizes (0: it does not take them): a block holds all of
// a head's columns, so Dv * P <= 1024, and a lane at most 32 rows.
RB_EXPORT int rb_delta_step_lanes(int D, int Dv, int n_rows) {
  if (D <= 0 || Dv <= 0 || n_rows > 64) return 0;
  int P = 32;
  while (P > 1 && (Dv * P > 1024 || (D + P - 1) / P < 4)) P >>= 1;
  if (Dv * P > 1024 || (D + P - 1) / P > 32) return 0;
  return P;
}

// A decode step's delta rule in one launch (see the kernel).  proj: float32 rows [q | k | v | g | b | a] of the stacked
// product; out: [rows, H * Dv] in float32 or bfloat16.
RB_EXPORT int rb_delta_step(void* out, int out_dtype, const float* proj, int64_t ld, int g_off, int b_off, int a_off,
                            const float* taps, const float* A_log, const float* dt_bias, const float* norm_w, float* state,
                            float* tail, const int* tok_slot, const int* tok_pos, int n_rows, int H, int G, int D, int Dv, int K,
                            float q_scale, float unit_eps, float norm_eps, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  const int P = rb_delta_step_lanes(D, Dv, n_rows);
  RB_REQUIRE(P > 0 && H > 0 && G > 0 && H % G == 0 && K >= 1 && (K == 1 || tail != nullptr),
             "rb_delta_step: sizes H=%d G=%d D=%d Dv=%d taps=%d rows=%d are not taken", H, G, D, Dv, K, n_rows);
  const int per = (D + P - 1) / P;
  const int threads = (Dv * P + 31) / 32 * 32;
  const size_t smem = (size_t)(2 * D + Dv) * sizeof(float);
  const dim3 grid(n_rows, H);
  const int bf16 = out_dtype == RB_BF16 ? 1 : 0;
  RB_REQUIRE(out_dtype == RB_BF16 || out_dtype == RB_F32, "rb_delta_step: unknown dtype %d", out_dtype);
  if (per <= 16)
    RB_LAUNCH("delta_step_kernel", (delta_step_kernel<16>), grid, threads, smem, stream, out, bf16, proj, ld, g_off, b_off, a_off, taps,
              A_log, dt_bias, norm_w, state, tail, tok_slot, tok_pos, H, G, D, Dv, K, P, q_scale, unit_eps, norm_eps);
  else
    RB_LAUNCH("delta_step_kernel", (delta_step_kernel<32>), grid, threads, smem, stream, out, bf16, proj, ld, g_off, b_off, a_off, taps,
              A_log, dt_bias, norm_w, state, tail, tok_slot, tok_pos, H, G, D, Dv, K, P, q_scale, unit_eps, norm_eps);
  RB_CHECK_LAUNCH("rb_delta_step");
  return 0;
}
