// Routing of a mixture of experts, all in 32-bit.
//
// jv_moe_route, one warp per token, from the router logits z = W_router x (a product made before it, with 32-bit
// accumulation and a 32-bit result):  s = softmax(z) over all experts, or sigmoid(z) of each (`scoring` 1); with groups, a
// group's score is its largest s, or the sum of its two largest (`group_mode` 1), and only experts of the
// `keep` best groups stay; the `top` largest s among those are chosen, largest first (lowest index on a tie);
// weight = s (divided by the chosen scores' sum plus `renorm_eps` if `renorm`), times `weight_scale`.
//
// jv_moe_align, one block: puts the (token, choice) pairs in the order of their experts, every expert's run
// padded to a multiple of `tile` rows so that a row tile of the grouped products belongs to one expert:
//   sorted_token[pos] = token (-1: padding), pos_of[token*top + k] = pos, tile_expert[tile] = expert (-1: unused),
//   tile_expert[max_tiles] = number of tiles in use (they are the first ones).
// Which of an expert's rows a pair gets depends on the order of arrival; no result depends on it, since every
// row of a product is computed alone.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int ROUTE_WARPS = 4;

__global__ void __launch_bounds__(ROUTE_WARPS * 32) moe_route_kernel(
    const float* __restrict__ z, int z_stride, int n, int experts, int top, int groups,
    int keep, int renorm, int scoring, int group_mode, float renorm_eps, float weight_scale,
    int* __restrict__ ids, float* __restrict__ weights) {
  extern __shared__ float smem[];                 // [ROUTE_WARPS][experts] scores, [ROUTE_WARPS][groups] group scores
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= n) return;
  float* s = smem + (size_t)warp * (experts + groups);
  float* gs = s + experts;
  for (int e = lane; e < experts; e += 32) s[e] = z[(size_t)t * z_stride + e];
  __syncwarp();
  if (scoring == 1) {
    for (int e = lane; e < experts; e += 32) s[e] = 1.f / (1.f + expf(-s[e]));
  } else {
    float mx = -INFINITY;
    for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, s[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) sum += expf(s[e] - mx);
    sum = warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < experts; e += 32) s[e] = expf(s[e] - mx) / sum;
  }
  __syncwarp();
  const int per = experts / groups;
  if (groups > 1) {
    for (int g = lane; g < groups; g += 32) {
      float b = -1.f, b2 = -1.f;                  // the largest and the second largest score of the group
      for (int j = 0; j < per; ++j) {
        const float v = s[g * per + j];
        if (v > b) { b2 = b; b = v; }
        else if (v > b2) b2 = v;
      }
      gs[g] = (group_mode == 1 && per > 1) ? b + b2 : b;
    }
    __syncwarp();
    // keep the best `keep` groups: a kept group's score is made negative minus one, so it is not found again
    for (int it = 0; it < keep; ++it) {
      float bv = -1.f; int bi = 0x7fffffff;
      for (int g = lane; g < groups; g += 32)
        if (gs[g] > bv) { bv = gs[g]; bi = g; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (lane == 0 && bi != 0x7fffffff) gs[bi] = -2.f;
      __syncwarp();
    }
  }
  float chosen_sum = 0.f;
  for (int it = 0; it < top; ++it) {
    float bv = -1.f; int bi = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const bool allowed = groups <= 1 || gs[e / per] == -2.f;
      const float v = s[e];
      if (allowed && v > bv) { bv = v; bi = e; }      // ascending e: the lowest index wins a tie within a lane
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi == 0x7fffffff) { bi = 0; bv = 0.f; }      // fewer allowed experts than `top`: refused by the host
    if (lane == 0) {
      ids[(size_t)t * top + it] = bi;
      weights[(size_t)t * top + it] = bv;
      s[bi] = -1.f;                                    // taken
    }
    chosen_sum += bv;
    __syncwarp();
  }
  if (lane == 0) {
    for (int it = 0; it < top; ++it) {
      float w = weights[(size_t)t * top + it];
      if (renorm) w /= (chosen_sum + renorm_eps);
      weights[(size_t)t * top + it] = w * weight_scale;
    }
  }
}

__global__ void __launch_bounds__(1024) moe_align_kernel(const int* __restrict__ ids, int pairs, int top, int experts,
                                                         int tile, int max_tiles, int* __restrict__ sorted_token,
                                                         int* __restrict__ pos_of, int* __restrict__ tile_expert,
                                                         int* __restrict__ status) {
  extern __shared__ int sh[];                    // [experts] counts, [experts] first row, [experts] cursor
  int* count = sh;
  int* first = sh + experts;
  int* cursor = first + experts;
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
  for (int i = threadIdx.x; i < max_tiles * tile; i += blockDim.x) sorted_token[i] = -1;
  for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) tile_expert[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
    else atomicOr(status, JV_STATUS_BAD_ROW);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int row = 0;
    for (int e = 0; e < experts; ++e) {
      first[e] = row;
      const int tiles = (count[e] + tile - 1) / tile;
      for (int k = 0; k < tiles; ++k) tile_expert[row / tile + k] = e;
      row += tiles * tile;
    }
    tile_expert[max_tiles] = row / tile;          // the row tiles in use are the first this many
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e < 0 || e >= experts) { pos_of[i] = -1; continue; }
    const int pos = first[e] + atomicAdd(&cursor[e], 1);
    sorted_token[pos] = i / top;
    pos_of[i] = pos;
  }
}

// out[pos_of[i], :] = x[i / top, :] for every (token, choice) pair i: the rows in the order of their experts.
template <typename T>
__global__ void moe_gather_rows_kernel(const T* __restrict__ x, int x_stride, const int* __restrict__ pos_of, int top,
                                       T* __restrict__ out, int out_rows, int width) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const int pos = pos_of[i];
  if (pos < 0 || pos >= out_rows) return;
  const T* src = x + (size_t)(i / top) * x_stride;
  T* dst = out + (size_t)pos * width;
  if (sizeof(T) == 2 && width % 8 == 0 && x_stride % 8 == 0) {
    for (int c = threadIdx.x; c < width / 8; c += blockDim.x)
      reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
  } else {
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = src[c];
  }
}
}  // namespace

// x: [n, width] rows of x_stride; pos_of: [pairs]; out: [out_rows, width] (rows that no pair names are left alone).
JV_EXPORT int jv_moe_gather_rows(const void* x, int dtype, int x_stride, const int* pos_of, int pairs, int top, void* out,
                                 int out_rows, int width, cudaStream_t stream) {
  if (pairs == 0) return JV_OK;
  JV_DISPATCH_DTYPE(dtype, T, return jv_launch(moe_gather_rows_kernel<T>, dim3(pairs), dim3(128), 0, stream, (const T*)x,
                                               x_stride, pos_of, top, (T*)out, out_rows, width));
  return JV_ERR_UNSUPPORTED;
}

// z: [n, experts] float rows of z_stride elements; ids: [n, top] int32; weights: [n, top] float.
JV_EXPORT int jv_moe_route(const float* z, int z_stride, int n, int experts, int top, int groups, int keep, int renorm,
                           int scoring, int group_mode, float renorm_eps, float weight_scale, int* ids, float* weights,
                           cudaStream_t stream) {
  if (n == 0) return JV_OK;
  if (experts < 1 || top < 1 || top > experts || groups < 1 || experts % groups || keep < 1 || keep > groups ||
      top > keep * (experts / groups))
    return JV_ERR_UNSUPPORTED;
  const size_t smem = sizeof(float) * ROUTE_WARPS * (size_t)(experts + groups);
  if (smem > 48 * 1024) return JV_ERR_UNSUPPORTED;
  const int blocks = (n + ROUTE_WARPS - 1) / ROUTE_WARPS;
  return jv_launch(moe_route_kernel, dim3(blocks), dim3(ROUTE_WARPS * 32), smem, stream, z, z_stride, n, experts, top,
                   groups, keep, renorm, scoring, group_mode, renorm_eps, weight_scale, ids, weights);
}

// ids: [pairs] experts of the (token, choice) pairs, pairs = n * top; sorted_token: [max_tiles * tile];
// pos_of: [pairs]; tile_expert: [max_tiles + 1], max_tiles >= pairs / tile + experts.
JV_EXPORT int jv_moe_align(const int* ids, int pairs, int top, int experts, int tile, int max_tiles, int* sorted_token,
                           int* pos_of, int* tile_expert, int* status, cudaStream_t stream) {
  if (pairs == 0) return JV_OK;
  if (tile < 1 || (long long)max_tiles * tile < (long long)pairs + (long long)experts * (tile - 1) ||
      experts * 3 * sizeof(int) > 48 * 1024)
    return JV_ERR_UNSUPPORTED;
  return jv_launch(moe_align_kernel, dim3(1), dim3(1024), (size_t)experts * 3 * sizeof(int), stream, ids, pairs, top,
                   experts, tile, max_tiles, sorted_token, pos_of, tile_expert, status);
}
