// Query/key/value preparation head by head, fused with the write of the new keys and values into the paged cache.
// One warp handles one head of one token of a packed projection row `proj` (queries at q_off, keys at k_off, values at
// v_off; element offsets).  Every step is optional and all arithmetic is 32-bit (sums of squares, angles, cosines,
// sines):
//
//   queries, keys   u <- u * rsqrt(mean(u^2) + eps) * weight[D]          one weight vector shared by all heads
//                   rotation of the first rot_dim elements of the head by position * freq[j]; the rest passes
//   values          v <- v * rsqrt(mean(v^2) + eps)                      no weight
//                   rotation of the first v_rot_dim elements by position * v_freq[j]: a value that carries its own
//                   position, so that the summed output can be turned back by the query's position (jv_head_rotate)
//
// The pairs of a rotation are (j, j + dims/2) ("halves") or (2j, 2j + 1) (`interleaved`); the pair (u, v) becomes
// (u cos a - v sin a, v cos a + u sin a).  Queries go to q_out [n, Hq*D]; keys to k_cache[page, slot, key head, :D];
// values to v_cache[page, slot, value head, :DV].
//
// jv_head_rotate turns every head of rows [n, heads*dim] by sign * position * freq[j] (in place or into `out`).
//
// jv_rms_rows: out[t, :] = in[t, :width] * rsqrt(mean(in[t, :width]^2) + eps) * weight, for rows that are a column
// range of a wider product (the normed latent that a second product reads).
#include "common.cuh"

namespace {
constexpr int WARPS = 4;

struct HeadPrepareParams {
  const void* proj; long long row_stride; int q_off, k_off, v_off;
  void* q_out;
  const int* positions; const int* token_entry; const int* block_table; int table_width;
  const float* freq; int rot_dim;
  const float* v_freq; int v_rot_dim;
  int interleaved;
  const void* q_norm_w; const void* k_norm_w; float eps;
  int v_norm;
  void* k_cache; void* v_cache;
  int n, n_q_heads, n_k_heads, n_v_heads, key_dim, value_dim, page_size, num_pages;
  int* status;
};

// One head: dim elements at src -> dst; optional unit norm (with a weight, or none), optional rotation of the first
// `rot` elements.  The whole warp calls it.
template <typename T, typename TW>
__device__ __forceinline__ void prepare_head(const T* __restrict__ src, T* __restrict__ dst, int dim, bool normed,
                                             const TW* __restrict__ w, float eps, const float* __restrict__ freq, int rot,
                                             int interleaved, float pos, int lane) {
  float inv = 1.f;
  if (normed) {
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) { const float v = to_f32(src[d]); ss += v * v; }
    inv = rsqrtf(warp_sum(ss) / (float)dim + eps);
  }
  const int half = rot >> 1;
  for (int j = lane; j < half; j += 32) {
    const int i0 = interleaved ? 2 * j : j, i1 = interleaved ? 2 * j + 1 : j + half;
    float u = to_f32(src[i0]) * inv, v = to_f32(src[i1]) * inv;
    if (w != nullptr) { u *= to_f32(w[i0]); v *= to_f32(w[i1]); }
    float sn, cs;
    sincosf(pos * freq[j], &sn, &cs);
    dst[i0] = from_f32<T>(u * cs - v * sn);
    dst[i1] = from_f32<T>(v * cs + u * sn);
  }
  for (int d = rot + lane; d < dim; d += 32) {
    float u = to_f32(src[d]) * inv;
    if (w != nullptr) u *= to_f32(w[d]);
    dst[d] = from_f32<T>(u);
  }
}

template <typename T, typename TW>
__global__ void __launch_bounds__(32 * WARPS) head_prepare_kernel(const HeadPrepareParams p) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const bool writes = p.k_cache != nullptr;
  const int per_token = p.n_q_heads + (writes ? p.n_k_heads + p.n_v_heads : 0);
  const long long item = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (item >= (long long)p.n * per_token) return;
  const int t = (int)(item / per_token);
  int h = (int)(item - (long long)t * per_token);
  const int posi = p.positions[t];
  const float pos = (float)posi;
  const T* row = (const T*)p.proj + (size_t)t * p.row_stride;
  if (h < p.n_q_heads) {
    prepare_head<T, TW>(row + p.q_off + (size_t)h * p.key_dim, (T*)p.q_out + ((size_t)t * p.n_q_heads + h) * p.key_dim,
                        p.key_dim, p.q_norm_w != nullptr, (const TW*)p.q_norm_w, p.eps, p.freq, p.rot_dim, p.interleaved,
                        pos, lane);
    return;
  }
  h -= p.n_q_heads;
  const int entry = p.token_entry[t];
  const int page_idx = posi / p.page_size;
  const int page = (posi >= 0 && page_idx < p.table_width) ? p.block_table[(size_t)entry * p.table_width + page_idx] : -1;
  if (page < 0 || page >= p.num_pages) {
    if (lane == 0) atomicOr(p.status, JV_STATUS_BAD_PAGE);
    return;
  }
  const size_t slot = (size_t)page * p.page_size + (posi - page_idx * p.page_size);
  if (h < p.n_k_heads) {
    prepare_head<T, TW>(row + p.k_off + (size_t)h * p.key_dim, (T*)p.k_cache + (slot * p.n_k_heads + h) * p.key_dim,
                        p.key_dim, p.k_norm_w != nullptr, (const TW*)p.k_norm_w, p.eps, p.freq, p.rot_dim, p.interleaved,
                        pos, lane);
    return;
  }
  h -= p.n_k_heads;
  prepare_head<T, TW>(row + p.v_off + (size_t)h * p.value_dim, (T*)p.v_cache + (slot * p.n_v_heads + h) * p.value_dim,
                      p.value_dim, p.v_norm != 0, (const TW*)nullptr, p.eps, p.v_freq, p.v_rot_dim, p.interleaved, pos, lane);
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(32 * WARPS) head_rotate_kernel(const TI* in, long long in_stride, TO* out, long long out_stride,
                                                                const int* __restrict__ positions,
                                                                const float* __restrict__ freq, int rot, int interleaved,
                                                                float sign, int n, int heads, int dim) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (item >= (long long)n * heads) return;
  const int t = (int)(item / heads), h = (int)(item - (long long)t * heads);
  const float pos = sign * (float)positions[t];
  const TI* src = in + (size_t)t * in_stride + (size_t)h * dim;
  TO* dst = out + (size_t)t * out_stride + (size_t)h * dim;
  const int half = rot >> 1;
  for (int j = lane; j < half; j += 32) {
    const int i0 = interleaved ? 2 * j : j, i1 = interleaved ? 2 * j + 1 : j + half;
    const float u = to_f32(src[i0]), v = to_f32(src[i1]);
    float sn, cs;
    sincosf(pos * freq[j], &sn, &cs);
    dst[i0] = from_f32<TO>(u * cs - v * sn);
    dst[i1] = from_f32<TO>(v * cs + u * sn);
  }
  for (int d = rot + lane; d < dim; d += 32) dst[d] = from_f32<TO>(to_f32(src[d]));
}

template <typename T, typename TW>
__global__ void __launch_bounds__(128) rms_rows_kernel(const T* __restrict__ in, long long in_stride, T* __restrict__ out,
                                                       long long out_stride, const TW* __restrict__ w, float eps,
                                                       int width) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const T* src = in + (size_t)blockIdx.x * in_stride;
  T* dst = out + (size_t)blockIdx.x * out_stride;
  float ss = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) { const float v = to_f32(src[d]); ss += v * v; }
  const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + eps);
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float v = to_f32(src[d]) * inv;
    if (w != nullptr) v *= to_f32(w[d]);
    dst[d] = from_f32<T>(v);
  }
}
}  // namespace

// proj: [n, row_stride] of `dtype`; q_out: [n, n_q_heads*key_dim] of `dtype`; q_norm_w, k_norm_w: [key_dim] of
// `w_dtype` or null; freq: [rot_dim/2] float or null (rot_dim 0); v_freq: [v_rot_dim/2] or null; v_norm: values
// are unit-normed (no weight); caches as for jv_attn_prepare, both null: queries only.
JV_EXPORT int jv_head_prepare(const void* proj, int dtype, long long row_stride, int q_off, int k_off, int v_off,
                              void* q_out, const int* positions, const int* token_entry, const int* block_table,
                              int table_width, const float* freq, int rot_dim, const float* v_freq, int v_rot_dim,
                              int interleaved, const void* q_norm_w, const void* k_norm_w, int w_dtype, float eps,
                              int v_norm, void* k_cache, void* v_cache, int n, int n_q_heads, int n_k_heads,
                              int n_v_heads, int key_dim, int value_dim, int page_size, int num_pages, int* status,
                              cudaStream_t stream) {
  if (n == 0) return JV_OK;
  if (rot_dim < 0 || rot_dim > key_dim || (rot_dim & 1) || (rot_dim > 0 && freq == nullptr) || v_rot_dim < 0 ||
      v_rot_dim > value_dim || (v_rot_dim & 1) || (v_rot_dim > 0 && v_freq == nullptr) || key_dim < 1 || value_dim < 1 ||
      page_size < 1 || (k_cache == nullptr) != (v_cache == nullptr))
    return JV_ERR_UNSUPPORTED;
  HeadPrepareParams p;
  p.proj = proj; p.row_stride = row_stride; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.q_out = q_out;
  p.positions = positions; p.token_entry = token_entry; p.block_table = block_table; p.table_width = table_width;
  p.freq = freq; p.rot_dim = rot_dim; p.v_freq = v_freq; p.v_rot_dim = v_rot_dim; p.interleaved = interleaved ? 1 : 0;
  p.q_norm_w = q_norm_w; p.k_norm_w = k_norm_w; p.eps = eps; p.v_norm = v_norm ? 1 : 0; p.k_cache = k_cache;
  p.v_cache = v_cache; p.n = n; p.n_q_heads = n_q_heads; p.n_k_heads = n_k_heads; p.n_v_heads = n_v_heads;
  p.key_dim = key_dim; p.value_dim = value_dim; p.page_size = page_size; p.num_pages = num_pages; p.status = status;
  const long long items = (long long)n * (n_q_heads + (k_cache != nullptr ? n_k_heads + n_v_heads : 0));
  const dim3 grid((unsigned)((items + WARPS - 1) / WARPS));
  JV_DISPATCH_DTYPE(dtype, T, {
    if (w_dtype == 0) return jv_launch(head_prepare_kernel<T, float>, grid, dim3(32 * WARPS), 0, stream, p);
    if (w_dtype == 1) return jv_launch(head_prepare_kernel<T, __nv_bfloat16>, grid, dim3(32 * WARPS), 0, stream, p);
  });
  return JV_ERR_UNSUPPORTED;
}

// in: [n, in_stride] of in_dtype, out: [n, out_stride] of out_dtype (may be `in`, with equal types), heads of `dim`
// elements side by side; the first `rot` elements of every head turn by sign * position * freq[j].
JV_EXPORT int jv_head_rotate(const void* in, int in_dtype, long long in_stride, void* out, int out_dtype,
                             long long out_stride, const int* positions, const float* freq, int rot, int interleaved,
                             float sign, int n, int heads, int dim, cudaStream_t stream) {
  if (n == 0 || heads == 0) return JV_OK;
  if (rot < 0 || rot > dim || (rot & 1) || (rot > 0 && freq == nullptr)) return JV_ERR_UNSUPPORTED;
  const long long items = (long long)n * heads;
  const dim3 grid((unsigned)((items + WARPS - 1) / WARPS));
  JV_DISPATCH_DTYPE(in_dtype, TI, JV_DISPATCH_DTYPE(out_dtype, TO,
      return jv_launch(head_rotate_kernel<TI, TO>, grid, dim3(32 * WARPS), 0, stream, (const TI*)in, in_stride, (TO*)out,
                       out_stride, positions, freq, rot, interleaved ? 1 : 0, sign, n, heads, dim)));
  return JV_ERR_UNSUPPORTED;
}

// in: [n, in_stride], out: [n, out_stride] of `dtype`; w: [width] of w_dtype or null.
JV_EXPORT int jv_rms_rows(const void* in, long long in_stride, void* out, long long out_stride, int dtype, const void* w,
                          int w_dtype, float eps, int n, int width, cudaStream_t stream) {
  if (n == 0) return JV_OK;
  if (width < 1) return JV_ERR_UNSUPPORTED;
  JV_DISPATCH_DTYPE(dtype, T, JV_DISPATCH_DTYPE(w_dtype, TW,
      return jv_launch(rms_rows_kernel<T, TW>, dim3(n), dim3(128), 0, stream, (const T*)in, in_stride, (T*)out, out_stride,
                       (const TW*)w, eps, width)));
  return JV_ERR_UNSUPPORTED;
}
