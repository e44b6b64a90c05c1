// Several residual streams per token (hyper-connections) and the glue between two sublayers.
//
// The residual state of a token is s rows X[t][0..s-1][0..E-1] (float32).  A sublayer reads the
// mix u = sum_k in[k] X_k through an RMS norm, and its result y is written back to all streams at
// once from the old ones:  X'_j = sum_k mix[k][j] X_k + out[j] * y.   With s = 1, in = out = mix = 1
// this is the ordinary residual sum.
//
// One kernel does everything that lies between the products of two sublayers, one block per token:
//   1. y: the sublayer's result, or the mean of up to MAX_Y results each under its own RMS norm
//      (mixers that run side by side);
//   2. the write into the streams (skipped without y);
//   3. the next sublayer's read and its norm (skipped without a next sublayer).
// Every part can also run alone, which is how the fused call is tested against its pieces.
// All arithmetic is float32.
#include "rb_common.cuh"

namespace {

constexpr int MAX_STREAMS = 16;
constexpr int MAX_Y = 4;

struct StreamStepArgs {
  float* X;                      // [T, s, E]; null: only the results are combined (into y_out)
  int s, E;
  const float* y[MAX_Y];         // [T, E] each; n_y == 0: nothing is written
  const float* y_norm[MAX_Y];    // [E] each, or null: y[0] is taken as it is
  int n_y;
  const float* mix;              // [s, s], indexed [from, to]
  const float* w_out;            // [s]
  const float* w_in;             // [s] of the NEXT read, or null
  const float* norm_w;           // [E] of the next read's norm
  float eps;
  void* h_out;                   // [T, E] in the compute dtype
  float* y_out;                  // optional [T, E]: the combined y, for whoever wants it alone
};

// S > 0: the number of streams is known when the kernel is compiled (loops unroll without tests); S == 0: any
// number up to MAX_STREAMS.  VEC == 4: rows are read and written four values at a time (E a multiple of 4,
// 16-byte aligned pointers).
template <typename TO, int S, int VEC>
__global__ void __launch_bounds__(256) stream_step_kernel(StreamStepArgs a) {
  rb_pdl_launch_dependents();
  constexpr int SS = S > 0 ? S : MAX_STREAMS;
  __shared__ float scratch[33];
  __shared__ float s_mix[SS * SS], s_out[SS], s_in[SS];
  extern __shared__ __align__(16) float urow[];     // E floats: the next read's mix
  const int t = blockIdx.x, s = S > 0 ? S : a.s, E = a.E;
  // the small tables are weights: they do not depend on the kernel before
  if (a.n_y > 0 && a.mix != nullptr)
    for (int i = threadIdx.x; i < s * s; i += blockDim.x) s_mix[i] = a.mix[i];
  if (threadIdx.x < s) {
    s_out[threadIdx.x] = (a.n_y > 0 && a.w_out != nullptr) ? a.w_out[threadIdx.x] : 0.f;
    s_in[threadIdx.x] = a.w_in != nullptr ? a.w_in[threadIdx.x] : 0.f;
  }
  rb_pdl_wait();
  // 1. factors of the results' norms
  float yfac[MAX_Y];
  const bool normed = a.n_y > 0 && a.y_norm[0] != nullptr;
#pragma unroll
  for (int k = 0; k < MAX_Y; ++k) {
    yfac[k] = 1.f;
    if (normed && k < a.n_y) {
      const float* yr = a.y[k] + (int64_t)t * E;
      float ss = 0.f;
      if (VEC == 4) {
        for (int e = threadIdx.x * 4; e < E; e += blockDim.x * 4) {
          const float4 v = *reinterpret_cast<const float4*>(yr + e);
          ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
      } else {
        for (int e = threadIdx.x; e < E; e += blockDim.x) ss += yr[e] * yr[e];
      }
      ss = rb_block_sum(ss, scratch);
      yfac[k] = 1.0f / sqrtf(ss / (float)E + a.eps);
    }
  }
  __syncthreads();
  float* Xt = a.X + (int64_t)t * s * E;
  float ss = 0.f;
  for (int e = threadIdx.x * VEC; e < E; e += blockDim.x * VEC) {
    float xs[SS][VEC];
#pragma unroll
    for (int k = 0; k < SS; ++k) {
      if (k < s && a.X != nullptr) {
        if (VEC == 4) {
          const float4 v = *reinterpret_cast<const float4*>(Xt + (int64_t)k * E + e);
          xs[k][0] = v.x; xs[k][1] = v.y; xs[k][2] = v.z; xs[k][VEC - 1] = v.w;
        } else {
          xs[k][0] = Xt[(int64_t)k * E + e];
        }
      } else {
#pragma unroll
        for (int v = 0; v < VEC; ++v) xs[k][v] = 0.f;
      }
    }
    if (a.n_y > 0) {
      float y[VEC];
      if (normed) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) y[v] = 0.f;
#pragma unroll
        for (int k = 0; k < MAX_Y; ++k)
          if (k < a.n_y) {
#pragma unroll
            for (int v = 0; v < VEC; ++v) y[v] += a.y[k][(int64_t)t * E + e + v] * yfac[k] * a.y_norm[k][e + v];
          }
#pragma unroll
        for (int v = 0; v < VEC; ++v) y[v] *= 1.0f / (float)a.n_y;
      } else {
#pragma unroll
        for (int v = 0; v < VEC; ++v) y[v] = a.y[0][(int64_t)t * E + e + v];
      }
      if (a.y_out != nullptr) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) a.y_out[(int64_t)t * E + e + v] = y[v];
      }
      if (a.X == nullptr) continue;
      float nx[SS][VEC];
#pragma unroll
      for (int j = 0; j < SS; ++j) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          float acc = 0.f;
          if (j < s) {
#pragma unroll
            for (int k = 0; k < SS; ++k)
              if (k < s) acc = fmaf(s_mix[k * s + j], xs[k][v], acc);
            acc = fmaf(s_out[j], y[v], acc);
          }
          nx[j][v] = acc;
        }
      }
#pragma unroll
      for (int j = 0; j < SS; ++j) {
        if (j >= s) continue;
#pragma unroll
        for (int v = 0; v < VEC; ++v) xs[j][v] = nx[j][v];
        if (VEC == 4) *reinterpret_cast<float4*>(Xt + (int64_t)j * E + e) = make_float4(nx[j][0], nx[j][1], nx[j][2], nx[j][VEC - 1]);
        else Xt[(int64_t)j * E + e] = nx[j][0];
      }
    }
    if (a.w_in != nullptr) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        float u = 0.f;
#pragma unroll
        for (int k = 0; k < SS; ++k)
          if (k < s) u = fmaf(s_in[k], xs[k][v], u);
        urow[e + v] = u;
        ss += u * u;
      }
    }
  }
  if (a.w_in == nullptr) return;
  ss = rb_block_sum(ss, scratch);
  const float r = 1.0f / sqrtf(ss / (float)E + a.eps);
  TO* h = (TO*)a.h_out + (int64_t)t * E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) h[e] = rb_from_float<TO>(urow[e] * a.norm_w[e] * r);
}

// X[t][k][:] = x[t][:] for every stream k
__global__ void streams_expand_kernel(float* __restrict__ X, const float* __restrict__ x, int s, int E) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int t = blockIdx.x;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const float v = x[(int64_t)t * E + e];
    for (int k = 0; k < s; ++k) X[((int64_t)t * s + k) * E + e] = v;
  }
}

// out[r][:] = sum_k X[r][k][:], streams added in ascending order
__global__ void streams_sum_kernel(float* __restrict__ out, const float* __restrict__ X, int s, int E) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int t = blockIdx.x;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float v = 0.f;
    for (int k = 0; k < s; ++k) v += X[((int64_t)t * s + k) * E + e];
    out[(int64_t)t * E + e] = v;
  }
}

}  // namespace

RB_EXPORT int rb_streams_max() { return MAX_STREAMS; }
RB_EXPORT int rb_streams_max_results() { return MAX_Y; }

// y: n_y pointers (host array) to [T, E] float32; y_norm: n_y pointers to [E] weights, or null for a
// single result taken as it is.  w_in null: no next read.  n_y == 0: only the read.
RB_EXPORT int rb_stream_step(float* X, int T, int s, int E, const float* const* y, const float* const* y_norm, int n_y,
                             const float* mix, const float* w_out, const float* w_in, const float* norm_w, float eps,
                             void* h_out, int h_dtype, float* y_out, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(s >= 1 && s <= MAX_STREAMS, "rb_stream_step: %d streams (1..%d are built)", s, MAX_STREAMS);
  RB_REQUIRE(n_y >= 0 && n_y <= MAX_Y, "rb_stream_step: %d results to combine (0..%d are built)", n_y, MAX_Y);
  RB_REQUIRE(E > 0 && (size_t)E * 4 <= 200 * 1024, "rb_stream_step: width %d", E);
  RB_REQUIRE(n_y == 0 || X == nullptr || (mix != nullptr && w_out != nullptr), "rb_stream_step: a write needs mix and out weights");
  RB_REQUIRE(X != nullptr || (y_out != nullptr && w_in == nullptr && n_y > 0), "rb_stream_step: without a state only results are combined");
  RB_REQUIRE(n_y <= 1 || y_norm != nullptr, "rb_stream_step: several results are combined under their norms");
  RB_REQUIRE(w_in == nullptr || (norm_w != nullptr && h_out != nullptr), "rb_stream_step: a read needs its norm and an output");
  StreamStepArgs a{};
  a.X = X; a.s = s; a.E = E; a.n_y = n_y;
  for (int k = 0; k < n_y; ++k) {
    a.y[k] = y[k];
    a.y_norm[k] = y_norm != nullptr ? y_norm[k] : nullptr;
  }
  a.mix = mix; a.w_out = w_out; a.w_in = w_in; a.norm_w = norm_w; a.eps = eps; a.h_out = h_out; a.y_out = y_out;
  const size_t smem = w_in != nullptr ? (size_t)E * sizeof(float) : 0;
  bool vec = E % 4 == 0 && (uintptr_t)X % 16 == 0 && (uintptr_t)y_out % 16 == 0;
  for (int k = 0; k < n_y; ++k) vec = vec && (uintptr_t)a.y[k] % 16 == 0 && (uintptr_t)a.y_norm[k] % 16 == 0;
  vec = vec && (s <= 4 || s == 8);        // other numbers of streams take the kernel for any number, value by value
  const int per = vec ? 4 : 1;
  int threads = 64;
  while (threads < 256 && threads * per < E) threads *= 2;
#define LAUNCH(TO, S, V)                                                                                             \
  do {                                                                                                               \
    if (smem > 48 * 1024)                                                                                            \
      RB_CUDA(cudaFuncSetAttribute(stream_step_kernel<TO, S, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    RB_LAUNCH("stream_step_kernel", (stream_step_kernel<TO, S, V>), T, threads, smem, stream, a);                    \
  } while (0)
#define BY_STREAMS(TO)                                                                                               \
  do {                                                                                                               \
    if (vec && s == 1) LAUNCH(TO, 1, 4);                                                                             \
    else if (vec && s == 2) LAUNCH(TO, 2, 4);                                                                        \
    else if (vec && s == 3) LAUNCH(TO, 3, 4);                                                                        \
    else if (vec && s == 4) LAUNCH(TO, 4, 4);                                                                        \
    else if (vec && s == 8) LAUNCH(TO, 8, 4);                                                                        \
    else LAUNCH(TO, 0, 1);                                                                                           \
  } while (0)
  if (h_dtype == RB_BF16) BY_STREAMS(__nv_bfloat16);
  else if (h_dtype == RB_F32) BY_STREAMS(float);
  else RB_FAIL("rb_stream_step: unknown dtype %d", h_dtype);
#undef BY_STREAMS
#undef LAUNCH
  RB_CHECK_LAUNCH("rb_stream_step");
  return 0;
}

RB_EXPORT int rb_streams_expand(float* X, const float* x, int T, int s, int E, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(s >= 1 && E > 0, "rb_streams_expand: bad sizes s=%d E=%d", s, E);
  RB_LAUNCH("streams_expand_kernel", (streams_expand_kernel), T, 256, 0, stream, X, x, s, E);
  RB_CHECK_LAUNCH("rb_streams_expand");
  return 0;
}

RB_EXPORT int rb_streams_sum(float* out, const float* X, int T, int s, int E, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(s >= 1 && E > 0, "rb_streams_sum: bad sizes s=%d E=%d", s, E);
  RB_LAUNCH("streams_sum_kernel", (streams_sum_kernel), T, 256, 0, stream, out, X, s, E);
  RB_CHECK_LAUNCH("rb_streams_sum");
  return 0;
}
