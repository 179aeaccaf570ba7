// Dynamic-tanh norm and the residual updates that go with it, all on the 32-bit stream.
//
//   jv_gated_add_dyt   h <- h + sigmoid(z + zb) * y      (y: a branch's output; the gate is optional, so is y)
//                      x  = tanh(alpha * h) * w + b      (optional: without w only the sum is made)
//                      One pass over the stream does both: the sum of the sublayer before and the norm of the
//                      sublayer after.  With `rows` only those rows are normed and h stays as it is (the final norm
//                      at the places whose logits are wanted).  The norm computes no mean and no variance, so a row
//                      needs no reduction and the kernel is a flat loop over elements.
//   jv_add_row         h[n, :] += vec                     (a learned vector added to every token)
//   jv_norm_mean2      out = c * (unit(a) * wa + unit(b) * wb), unit(y) = y / sqrt(mean(y^2) + eps) over a row: two
//                      mixers side by side, each normed before their mean is taken.
#include "common.cuh"
#include <math.h>

namespace {

template <typename Y, typename Z, typename W, typename O>
__global__ void __launch_bounds__(256) gated_add_dyt_kernel(float* __restrict__ h, const int* __restrict__ rows,
                                                            const Y* __restrict__ y, const Z* __restrict__ z,
                                                            long long z_stride, const W* __restrict__ zb, float alpha,
                                                            const W* __restrict__ w, const W* __restrict__ b,
                                                            O* __restrict__ out, int n_out, int n_total, int hidden,
                                                            int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)n_out * hidden;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const size_t i = idx / hidden;
    const int j = (int)(idx - i * hidden);
    size_t r = i;
    if (rows != nullptr) {
      const int rr = rows[i];
      if (rr < 0 || rr >= n_total) {
        if (j == 0) atomicOr(status, JV_STATUS_BAD_ROW);
        if (out != nullptr) out[idx] = from_f32<O>(0.f);
        continue;
      }
      r = (size_t)rr;
    }
    float v = h[r * hidden + j];
    if (y != nullptr) {
      float d = to_f32(y[r * hidden + j]);
      if (z != nullptr) d *= 1.f / (1.f + expf(-(to_f32(z[r * z_stride + j]) + to_f32(zb[j]))));
      v += d;
      if (rows == nullptr) h[r * hidden + j] = v;
    }
    if (out != nullptr) out[idx] = from_f32<O>(fmaf(tanhf(alpha * v), to_f32(w[j]), to_f32(b[j])));
  }
}

template <typename W>
__global__ void __launch_bounds__(256) add_row_kernel(float* __restrict__ h, const W* __restrict__ vec, size_t total,
                                                      int hidden) {
  pdl_trigger();
  pdl_wait();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride)
    h[idx] += to_f32(vec[idx % hidden]);
}

template <typename A, typename W>
__global__ void __launch_bounds__(256) norm_mean2_kernel(const A* __restrict__ a, const A* __restrict__ b,
                                                         const W* __restrict__ wa, const W* __restrict__ wb,
                                                         float* __restrict__ out, int hidden, float eps, float coef) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * hidden;
  float sa = 0.f, sb = 0.f;
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
    const float x = to_f32(a[base + j]), y = to_f32(b[base + j]);
    sa = fmaf(x, x, sa);
    sb = fmaf(y, y, sb);
  }
  sa = block_sum(sa, scratch);
  sb = block_sum(sb, scratch);
  const float ia = 1.f / sqrtf(sa / (float)hidden + eps), ib = 1.f / sqrtf(sb / (float)hidden + eps);
  for (int j = threadIdx.x; j < hidden; j += blockDim.x)
    out[base + j] = coef * (to_f32(a[base + j]) * ia * to_f32(wa[j]) + to_f32(b[base + j]) * ib * to_f32(wb[j]));
}

int grid_for(size_t total) {
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return (int)blocks;
}

}  // namespace

// h: [n_total, hidden] float; rows: [n_out] or null (n_out == n_total); y: [n_total, hidden] of dtype y_dtype or null;
// z: rows of z_stride elements of dtype z_dtype or null, zb: [hidden]; w, b, zb of dtype w_dtype (w null: no norm,
// out unused); out: [n_out, hidden] of dtype out_dtype.
JV_EXPORT int jv_gated_add_dyt(float* h, const int* rows, const void* y, int y_dtype, const void* z, int z_dtype,
                               long long z_stride, const void* zb, float alpha, const void* w, const void* b, int w_dtype,
                               void* out, int out_dtype, int n_out, int n_total, int hidden, int* status,
                               cudaStream_t stream) {
  const size_t total = (size_t)n_out * hidden;
  if (total == 0) return JV_OK;
  if (w == nullptr) out = nullptr;
  JV_DISPATCH_DTYPE(y_dtype, Y, JV_DISPATCH_DTYPE(z_dtype, Z, JV_DISPATCH_DTYPE(w_dtype, W, JV_DISPATCH_DTYPE(out_dtype, O,
      return jv_launch(gated_add_dyt_kernel<Y, Z, W, O>, dim3(grid_for(total)), dim3(256), 0, stream, h, rows, (const Y*)y,
                       (const Z*)z, z_stride, (const W*)zb, alpha, (const W*)w, (const W*)b, (O*)out, n_out, n_total,
                       hidden, status)))));
  return JV_ERR_UNSUPPORTED;
}

JV_EXPORT int jv_add_row(float* h, const void* vec, int dtype, int n, int hidden, cudaStream_t stream) {
  const size_t total = (size_t)n * hidden;
  if (total == 0) return JV_OK;
  JV_DISPATCH_DTYPE(dtype, W, return jv_launch(add_row_kernel<W>, dim3(grid_for(total)), dim3(256), 0, stream, h,
                                               (const W*)vec, total, hidden));
  return JV_ERR_UNSUPPORTED;
}

// a, b: [n, hidden] of dtype `dtype`; wa, wb: [hidden] of dtype `w_dtype`; out: [n, hidden] float.
JV_EXPORT int jv_norm_mean2(const void* a, const void* b, int dtype, const void* wa, const void* wb, int w_dtype, float* out,
                            int n, int hidden, float eps, float coef, cudaStream_t stream) {
  if (n == 0) return JV_OK;
  JV_DISPATCH_DTYPE(dtype, A, JV_DISPATCH_DTYPE(w_dtype, W, return jv_launch(
      norm_mean2_kernel<A, W>, dim3(n), dim3(hidden >= 1024 ? 256 : 128), 0, stream, (const A*)a, (const A*)b,
      (const W*)wa, (const W*)wb, out, hidden, eps, coef)));
  return JV_ERR_UNSUPPORTED;
}
