// What stands around the state scan of a Mamba-2 mixer (state-space duality): per head a state S [N, E] (N state
// channels, E value channels) with
//
//   dt  = softplus(dt_raw + dt_bias)                 a = exp(-exp(A_log) * dt)
//   S  <- a S + dt * B x^T                           y = S^T C + D x
//
// which is the update of csrc/recurrent.cu's state scan with the key dt * B, the query C and the decay a in every
// key channel.  B and C are shared by the heads of a group (head h uses group h / (heads / groups)).
//
// jv_mamba_prepare, one warp per (token, head): packed[t, h] = (C_g, dt * B_g, a) as float32 [3][N], from the
//   convolved rows xbc = [x | B | C] and the raw step sizes; softplus, both exponentials and the product with B in 32-bit.
// jv_mamba_finish, one block per (token, norm group): y = (o + D_h x) * silu(z), divided by the root mean square of its
//   norm group (inner / norm_groups elements), times the norm weight; 32-bit, written in the compute type.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int WARPS = 4;

template <typename T, typename TW>
__global__ void __launch_bounds__(32 * WARPS) mamba_prepare_kernel(const T* __restrict__ xbc, long long xbc_stride, int b_off,
                                                                  int c_off, const T* __restrict__ dt_raw,
                                                                  long long dt_stride, const TW* __restrict__ dt_bias,
                                                                  const TW* __restrict__ a_log, float* __restrict__ packed,
                                                                  int n, int heads, int groups, int state) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (item >= (long long)n * heads) return;
  const int t = (int)(item / heads), h = (int)(item - (long long)t * heads);
  const int g = h / (heads / groups);
  const float z = to_f32(dt_raw[(size_t)t * dt_stride + h]) + to_f32(dt_bias[h]);
  const float dt = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));             // softplus, no clamp
  const float a = expf(-expf(to_f32(a_log[h])) * dt);
  const T* B = xbc + (size_t)t * xbc_stride + b_off + (size_t)g * state;
  const T* C = xbc + (size_t)t * xbc_stride + c_off + (size_t)g * state;
  float* dst = packed + (size_t)item * 3 * state;
  for (int i = lane; i < state; i += 32) {
    dst[i] = to_f32(C[i]);
    dst[state + i] = dt * to_f32(B[i]);
    dst[2 * state + i] = a;
  }
}

// A thread keeps up to KEEP of its group's gated values in registers between the sum of squares and the write (a
// group of up to KEEP * blockDim elements is then read once); a longer group is formed twice.
constexpr int KEEP = 8;

template <typename T, typename TW>
__global__ void __launch_bounds__(1024) mamba_finish_kernel(const float* __restrict__ o, const T* __restrict__ x,
                                                            long long x_stride, const T* __restrict__ z, long long z_stride,
                                                            const TW* __restrict__ skip, const TW* __restrict__ w,
                                                            T* __restrict__ out, long long out_stride, float eps, int value_dim,
                                                            int group_size, int inner) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, first = blockIdx.y * group_size;
  const float* ot = o + (size_t)t * inner + first;
  const T* xt = x + (size_t)t * x_stride + first;
  const T* zt = z + (size_t)t * z_stride + first;
  auto gated = [&](int i) {
    const float zz = to_f32(zt[i]);
    return (ot[i] + to_f32(skip[(first + i) / value_dim]) * to_f32(xt[i])) * (zz / (1.f + expf(-zz)));
  };
  const bool kept = group_size <= KEEP * (int)blockDim.x;
  float ys[KEEP];
  float ss = 0.f;
  if (kept) {
#pragma unroll
    for (int u = 0; u < KEEP; ++u) {
      const int i = threadIdx.x + u * blockDim.x;
      ys[u] = i < group_size ? gated(i) : 0.f;
      ss += ys[u] * ys[u];
    }
  } else {
    for (int i = threadIdx.x; i < group_size; i += blockDim.x) { const float y = gated(i); ss += y * y; }
  }
  const float inv = rsqrtf(block_sum(ss, scratch) / (float)group_size + eps);
  T* dst = out + (size_t)t * out_stride + first;
  if (kept) {
#pragma unroll
    for (int u = 0; u < KEEP; ++u) {
      const int i = threadIdx.x + u * blockDim.x;
      if (i < group_size) dst[i] = from_f32<T>(ys[u] * inv * to_f32(w[first + i]));
    }
  } else {
    for (int i = threadIdx.x; i < group_size; i += blockDim.x) dst[i] = from_f32<T>(gated(i) * inv * to_f32(w[first + i]));
  }
}
}  // namespace

// xbc: rows of `dtype`, B at b_off and C at c_off ([groups][state] each); dt_raw: rows of `dtype`, [heads] used;
// dt_bias, a_log: [heads] of w_dtype; packed: float [n, heads, 3, state].
JV_EXPORT int jv_mamba_prepare(const void* xbc, int dtype, long long xbc_stride, int b_off, int c_off, const void* dt_raw,
                               long long dt_stride, const void* dt_bias, const void* a_log, int w_dtype, float* packed,
                               int n, int heads, int groups, int state, cudaStream_t stream) {
  if (n == 0) return JV_OK;
  if (heads < 1 || groups < 1 || heads % groups || state < 1) return JV_ERR_UNSUPPORTED;
  const long long items = (long long)n * heads;
  const dim3 grid((unsigned)((items + WARPS - 1) / WARPS));
  JV_DISPATCH_DTYPE(dtype, T, JV_DISPATCH_DTYPE(w_dtype, TW,
      return jv_launch(mamba_prepare_kernel<T, TW>, grid, dim3(32 * WARPS), 0, stream, (const T*)xbc, xbc_stride, b_off,
                       c_off, (const T*)dt_raw, dt_stride, (const TW*)dt_bias, (const TW*)a_log, packed, n, heads, groups,
                       state)));
  return JV_ERR_UNSUPPORTED;
}

// o: float [n, inner] (the scan's output); x, z: rows of `dtype`, [inner] used; skip: [heads] and w: [inner] of
// w_dtype; out: rows of `dtype`.  inner = heads * value_dim = norm_groups * group_size.
JV_EXPORT int jv_mamba_finish(const float* o, const void* x, long long x_stride, const void* z, long long z_stride,
                              int dtype, const void* skip, const void* w, int w_dtype, void* out, long long out_stride,
                              float eps, int n, int heads, int value_dim, int norm_groups, cudaStream_t stream) {
  if (n == 0) return JV_OK;
  const int inner = heads * value_dim;
  if (heads < 1 || value_dim < 1 || norm_groups < 1 || inner % norm_groups) return JV_ERR_UNSUPPORTED;
  // two elements a thread where the group allows: many warps hide the loads' latency when there are few tokens
  int threads = ((inner / norm_groups + 1) / 2 + 31) / 32 * 32;
  threads = threads < 32 ? 32 : threads > 1024 ? 1024 : threads;
  JV_DISPATCH_DTYPE(dtype, T, JV_DISPATCH_DTYPE(w_dtype, TW,
      return jv_launch(mamba_finish_kernel<T, TW>, dim3(n, norm_groups), dim3(threads), 0, stream, o, (const T*)x, x_stride,
                       (const T*)z, z_stride, (const TW*)skip, (const TW*)w, (T*)out, out_stride, eps, value_dim,
                       inner / norm_groups, inner)));
  return JV_ERR_UNSUPPORTED;
}
