// What stands between the projections of a latent attention and its attention kernel, and behind it.
//
// jv_latent_prepare, one block per token, from the product row  [ q heads (plain | rot) ... | latent | key part ]:
//   * the latent (first `latent_dim` elements of the down-projection) is divided by its root mean square, times
//     its norm weight, in 32-bit, and written to the token's place in the paged cache; the key part behind it is
//     rotated at the token's position and written behind the latent:  cache row = [ normed latent | rotated part ];
//   * the query row that the attention kernel reads is put together per head as [ q_latent | rotated q part ]:
//     the rotated part from the product row, q_latent (the head's plain query part times W_uk, made by a batched
//     product before this kernel) copied from [heads, n, latent_dim] if it is given there (else the product has
//     written it in place already).
// Rotation: element i of the part is paired with i + rot_dim/2 (or, `interleaved`, element 2i with 2i + 1); angle =
// position * inv_freq[i], cos and sin in 32-bit.  The down-projection may lie in rows of its own (`kv_row`).  A layer that reads another layer's cache passes no cache and only gets its queries made.
//
// jv_gate_heads: out[t, h*dv + d] = o[h, t, d] * sigmoid(g[t, h*dv + d])  (o as the batched product left it).
#include "common.cuh"
#include <math.h>

namespace {
struct PrepareParams {
  const void* row; int row_stride;      // product rows
  const void* kv_row; int kv_row_stride;   // rows that hold the down-projection at kv_off (the product rows themselves if null)
  int interleaved;                      // pairs of the rotation: (2i, 2i + 1) instead of (i, i + rot_dim / 2)
  int q_off, kv_off;                    // first column of the queries / of the down-projection (-1: none)
  const void* q_latent;                 // [heads, n, latent_dim] or null
  void* q_out; int q_out_stride;        // [n, heads * (latent_dim + rot_dim)]
  const int* positions; const int* token_entry; const int* block_table; int table_width;
  const float* inv_freq;                // [rot_dim / 2] or null (no rotation)
  const void* norm_w; float eps;
  void* cache;                          // [num_pages, page_size, latent_dim + rot_dim] or null
  int n, heads, plain_dim, rot_dim, latent_dim, page_size, num_pages;
  int* status;
};

template <typename T, typename TW>
__global__ void __launch_bounds__(128) latent_prepare_kernel(const PrepareParams p) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int pos = p.positions[t];
  const int half = p.rot_dim / 2, dk = p.latent_dim + p.rot_dim, dh = p.plain_dim + p.rot_dim;
  const T* row = (const T*)p.row + (size_t)t * p.row_stride;
  T* qo = (T*)p.q_out + (size_t)t * p.q_out_stride;

  // queries: the rotated part of every head, and the latent part if it has to be moved here
  for (int idx = tid; idx < p.heads * half; idx += blockDim.x) {
    const int hh = idx / half, i = idx - hh * half;
    const T* src = row + p.q_off + (size_t)hh * dh + p.plain_dim;
    const int i0 = p.interleaved ? 2 * i : i, i1 = p.interleaved ? 2 * i + 1 : i + half;
    float u = to_f32(src[i0]), v = to_f32(src[i1]);
    if (p.inv_freq != nullptr) {
      float s, c;
      sincosf((float)pos * p.inv_freq[i], &s, &c);
      const float a = u * c - v * s, b = v * c + u * s;
      u = a; v = b;
    }
    qo[(size_t)hh * dk + p.latent_dim + i0] = from_f32<T>(u);
    qo[(size_t)hh * dk + p.latent_dim + i1] = from_f32<T>(v);
  }
  if (p.q_latent != nullptr) {
    const T* ql = (const T*)p.q_latent;
    constexpr int V = 16 / sizeof(T);             // elements in 16 bytes
    if (p.latent_dim % V == 0 && dk % V == 0 && p.q_out_stride % V == 0 && ((uintptr_t)ql % 16) == 0 && ((uintptr_t)p.q_out % 16) == 0) {
      const int per = p.latent_dim / V;
      for (int idx = tid; idx < p.heads * per; idx += blockDim.x) {
        const int hh = idx / per, i = (idx - hh * per) * V;
        *reinterpret_cast<uint4*>(qo + (size_t)hh * dk + i) =
            *reinterpret_cast<const uint4*>(ql + ((size_t)hh * p.n + t) * p.latent_dim + i);
      }
    } else {
      for (int idx = tid; idx < p.heads * p.latent_dim; idx += blockDim.x) {
        const int hh = idx / p.latent_dim, i = idx - hh * p.latent_dim;
        qo[(size_t)hh * dk + i] = ql[((size_t)hh * p.n + t) * p.latent_dim + i];
      }
    }
  }
  if (p.cache == nullptr) return;

  // the token's cache row
  const int entry = p.token_entry[t];
  const int pi = pos / p.page_size;
  const int page = (pos >= 0 && pi < p.table_width) ? p.block_table[(size_t)entry * p.table_width + pi] : -1;
  const bool ok = page >= 0 && page < p.num_pages;
  if (!ok && tid == 0) atomicOr(p.status, JV_STATUS_BAD_PAGE);
  const T* kv = (p.kv_row != nullptr ? (const T*)p.kv_row + (size_t)t * p.kv_row_stride : row) + p.kv_off;
  float ss = 0.f;
  for (int i = tid; i < p.latent_dim; i += blockDim.x) { const float v = to_f32(kv[i]); ss += v * v; }
  ss = block_sum(ss, scratch);
  if (!ok) return;
  const float inv = rsqrtf(ss / (float)p.latent_dim + p.eps);
  T* dst = (T*)p.cache + ((size_t)page * p.page_size + (pos % p.page_size)) * dk;
  const TW* w = (const TW*)p.norm_w;
  for (int i = tid; i < p.latent_dim; i += blockDim.x) dst[i] = from_f32<T>(to_f32(kv[i]) * inv * to_f32(w[i]));
  for (int i = tid; i < half; i += blockDim.x) {
    const int i0 = p.interleaved ? 2 * i : i, i1 = p.interleaved ? 2 * i + 1 : i + half;
    float u = to_f32(kv[p.latent_dim + i0]), v = to_f32(kv[p.latent_dim + i1]);
    if (p.inv_freq != nullptr) {
      float s, c;
      sincosf((float)pos * p.inv_freq[i], &s, &c);
      const float a = u * c - v * s, b = v * c + u * s;
      u = a; v = b;
    }
    dst[p.latent_dim + i0] = from_f32<T>(u);
    dst[p.latent_dim + i1] = from_f32<T>(v);
  }
}

// eight bfloat16 elements a thread (dv a multiple of 8, 16-byte aligned rows)
__global__ void gate_heads_vec_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ g, int g_stride,
                                      __nv_bfloat16* __restrict__ out, int n, int heads, int dv) {
  pdl_trigger();
  pdl_wait();
  const int per = dv / 8;
  const size_t total = (size_t)n * heads * per;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const int d = (int)(i % per) * 8;
    const int hh = (int)((i / per) % heads);
    const size_t t = i / ((size_t)per * heads);
    uint4 a = *reinterpret_cast<const uint4*>(o + ((size_t)hh * n + t) * dv + d);
    if (g != nullptr) {
      const uint4 b = *reinterpret_cast<const uint4*>(g + t * g_stride + (size_t)hh * dv + d);
      __nv_bfloat162* ah = reinterpret_cast<__nv_bfloat162*>(&a);
      const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 x = __bfloat1622float2(ah[k]), y = __bfloat1622float2(bh[k]);
        ah[k] = __floats2bfloat162_rn(x.x * (1.f / (1.f + expf(-y.x))), x.y * (1.f / (1.f + expf(-y.y))));
      }
    }
    *reinterpret_cast<uint4*>(out + (t * heads + hh) * dv + d) = a;
  }
}

template <typename T>
__global__ void gate_heads_kernel(const T* __restrict__ o, const T* __restrict__ g, int g_stride, T* __restrict__ out,
                                  int n, int heads, int dv) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)n * heads * dv;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const int d = (int)(i % dv);
    const int hh = (int)((i / dv) % heads);
    const size_t t = i / ((size_t)dv * heads);
    float v = to_f32(o[((size_t)hh * n + t) * dv + d]);
    if (g != nullptr) v *= 1.f / (1.f + expf(-to_f32(g[t * g_stride + (size_t)hh * dv + d])));
    out[i] = from_f32<T>(v);
  }
}
}  // namespace

JV_EXPORT int jv_latent_prepare(const void* row, int dtype, int row_stride, int q_off, int kv_off, const void* q_latent,
                                void* q_out, int q_out_stride, const int* positions, const int* token_entry,
                                const int* block_table, int table_width, const float* inv_freq, const void* norm_w,
                                int norm_dtype, float eps, void* cache, int n, int heads, int plain_dim, int rot_dim,
                                int latent_dim, int page_size, int num_pages, const void* kv_row, int kv_row_stride,
                                int interleaved, int* status, cudaStream_t stream) {
  if (n == 0) return JV_OK;
  if (rot_dim % 2 || heads < 1 || latent_dim < 1) return JV_ERR_UNSUPPORTED;
  PrepareParams p;
  p.row = row; p.row_stride = row_stride; p.q_off = q_off; p.kv_off = kv_off; p.q_latent = q_latent;
  p.kv_row = kv_row; p.kv_row_stride = kv_row_stride; p.interleaved = interleaved ? 1 : 0;
  p.q_out = q_out; p.q_out_stride = q_out_stride; p.positions = positions; p.token_entry = token_entry;
  p.block_table = block_table; p.table_width = table_width; p.inv_freq = inv_freq; p.norm_w = norm_w; p.eps = eps;
  p.cache = kv_off >= 0 ? cache : nullptr; p.n = n; p.heads = heads; p.plain_dim = plain_dim; p.rot_dim = rot_dim;
  p.latent_dim = latent_dim; p.page_size = page_size; p.num_pages = num_pages; p.status = status;
  JV_DISPATCH_DTYPE(dtype, T, JV_DISPATCH_DTYPE(norm_dtype, TW,
      return jv_launch(latent_prepare_kernel<T, TW>, dim3(n), dim3(128), 0, stream, p)));
  return JV_ERR_UNSUPPORTED;
}

// o: [heads, n, dv]; g: rows of g_stride elements, [n, heads*dv] used, or null (no gate); out: [n, heads*dv].
JV_EXPORT int jv_gate_heads(const void* o, const void* g, int g_stride, void* out, int dtype, int n, int heads, int dv,
                            cudaStream_t stream) {
  if (n == 0) return JV_OK;
  long long blocks = ((long long)n * heads * dv + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == 1 && dv % 8 == 0 && g_stride % 8 == 0 && ((uintptr_t)o % 16) == 0 && ((uintptr_t)g % 16) == 0 &&
      ((uintptr_t)out % 16) == 0) {
    long long vblocks = ((long long)n * heads * (dv / 8) + 255) / 256;
    if (vblocks > 148 * 16) vblocks = 148 * 16;
    return jv_launch(gate_heads_vec_kernel, dim3((int)vblocks), dim3(256), 0, stream, (const __nv_bfloat16*)o,
                     (const __nv_bfloat16*)g, g_stride, (__nv_bfloat16*)out, n, heads, dv);
  }
  JV_DISPATCH_DTYPE(dtype, T, return jv_launch(gate_heads_kernel<T>, dim3((int)blocks), dim3(256), 0, stream,
                                               (const T*)o, (const T*)g, g_stride, (T*)out, n, heads, dv));
  return JV_ERR_UNSUPPORTED;
}
