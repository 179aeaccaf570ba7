// Paged causal attention over a latent cache on the tensor cores (mma.sync m16n8k16, bfloat16 operands, 32-bit
// accumulation, 32-bit softmax), for cache rows of any size that is a multiple of 8 up to 640: ONE key/value head
// whose key is the whole cache row [dk] and whose value is the row's first dv elements (dv <= 512), shared by all
// query heads.  It serves the row sizes that the kernels built for fixed head sizes do not take.
//
// Work item = (entry, first token of the tile); grid.y = head group; grid.z = key split (1 unless SPLIT).  A tile is
// 64 rows = (token, query head) pairs: row m -> token q_off + m / heads_per_tile, head hg * heads_per_tile +
// m % heads_per_tile.  Warp w works on rows (w & 3) * 16 .. + 16 and, of the output columns, on the part
// (w >> 2) * DVW .. + DVW (WD parts: a row's 512 output columns are more than one warp's registers hold; the two
// warps of a row each form the scores over half of k and exchange the partial sums through shared memory).  Keys come in chunks of 32 rows by cp.async, two buffers; the chunk in
// shared memory is the B operand of S = Q K^T as it lies (k contiguous) and, read through ldmatrix.trans, of
// O += P V: the row is loaded once for both.  Softmax is the running (max, sum) form in registers.
//
// SPLIT: work items are single tokens; split s covers key positions [s*split_size, (s+1)*split_size); it writes its
// unnormalised sums and (max, sum) to part_o / part_ml, and `latent_combine_kernel` merges the splits of a row in
// ascending order, so a result does not depend on what else is in the batch.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int BLOCK_M = 64, BLOCK_N = 32, PAD = 8;
constexpr int XCH_BYTES = 2 * 4 * 2 * 16 * 32 * 4;      // the exchange of partial scores between the two warps of a row

struct LatentParams {
  const __nv_bfloat16* q; int q_stride;
  __nv_bfloat16* out; int out_stride;
  float* part_o; float* part_ml;
  const __nv_bfloat16* cache;
  const int* block_table; int table_width;
  const int* cu_seqlens; const int* start_pos; const int* work;
  int n_heads, dk, dv, page_size, num_pages;
  float scale;
  int window;                    // the mask as one number (common.cuh, first_visible)
  const float* sink;             // [n_heads] or null: exp(sink) counts once in the softmax's denominator, with no value
  int tokens_per_tile, heads_per_tile, split_size, n_splits;
  int qstride_s, kstride_s;      // shared-memory row strides (elements) of the query tile and of a key chunk
  int* status;
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(a), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <int DVW, int WD, bool SPLIT>
__global__ void __launch_bounds__(128 * WD, 1) attn_latent_mma_kernel(const LatentParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);               // [BLOCK_M][qstride_s]
  __nv_bfloat16* Ks = Qs + BLOCK_M * p.qstride_s;                                // [2][BLOCK_N][kstride_s]
  float* Xs = reinterpret_cast<float*>(Ks + 2 * BLOCK_N * p.kstride_s);          // [2][4][2][16][32], only with WD == 2
  __shared__ int row_pos_s[BLOCK_M];
  constexpr int THREADS = 128 * WD;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rw = warp & 3, dw = warp >> 2;
  // the work list runs from an entry's first tile to its last: taken from the back, the tiles with the most keys
  // start first and the short ones fill the end of the launch
  const int item = SPLIT ? blockIdx.x : gridDim.x - 1 - blockIdx.x;
  const int entry = p.work[2 * item], q_off = p.work[2 * item + 1];
  const int hg = blockIdx.y;
  const int q_begin = p.cu_seqlens[entry];
  const int q_len = p.cu_seqlens[entry + 1] - q_begin;
  const int ctx = p.start_pos[entry];
  const int tokens_here = min(p.tokens_per_tile, q_len - q_off);
  if (tokens_here <= 0) return;
  int j_lo = first_visible(ctx + q_off, p.window), j_hi = ctx + q_off + tokens_here;      // keys [j_lo, j_hi)
  if (SPLIT) {
    j_lo = max(j_lo, (int)blockIdx.z * p.split_size);
    j_hi = min(j_hi, (blockIdx.z + 1) * p.split_size);
    if (j_lo >= j_hi) return;
  }
  const int dk = p.dk, qs = p.qstride_s, ks = p.kstride_s;
  // scores are kept times log2(e): the softmax's exponentials are powers of two (maxima in part_ml are in that scale too)
  const float scale_log2 = p.scale * 1.4426950408889634f;
  const int dkp = (dk + 15) & ~15;

  // ---- zero both key buffers once (columns that no copy writes, and rows that no key fills, must be finite)
  {
    uint4* z = reinterpret_cast<uint4*>(Ks);
    const int n16 = 2 * BLOCK_N * ks / 8;
    for (int i = tid; i < n16; i += THREADS) z[i] = make_uint4(0, 0, 0, 0);
  }
  // ---- rows: positions and query vectors
  if (tid < BLOCK_M) {
    const int t = tid / p.heads_per_tile, hh = hg * p.heads_per_tile + tid % p.heads_per_tile;
    row_pos_s[tid] = (t < tokens_here && hh < p.n_heads) ? ctx + q_off + t : -1;
  }
  for (int idx = tid; idx < BLOCK_M * (qs / 8); idx += THREADS) {
    const int m = idx / (qs / 8), c8 = (idx - m * (qs / 8)) * 8;
    const int t = m / p.heads_per_tile, hh = hg * p.heads_per_tile + m % p.heads_per_tile;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t < tokens_here && hh < p.n_heads && c8 < dk)
      v = *reinterpret_cast<const uint4*>(p.q + (size_t)(q_begin + q_off + t) * p.q_stride + (size_t)hh * dk + c8);
    *reinterpret_cast<uint4*>(Qs + m * qs + c8) = v;
  }
  __syncthreads();

  // a key row of the chunk is copied by THREADS / BLOCK_N threads, 16 bytes each a turn: one look at the block table a
  // thread and chunk
  auto load_chunk = [&](int j0, int buf) {
    constexpr int TPR = THREADS / BLOCK_N;
    const int n = tid / TPR, j = j0 + n;
    if (j < j_hi) {
      const int pi = j / p.page_size;
      const int page = pi < p.table_width ? p.block_table[(size_t)entry * p.table_width + pi] : -1;
      if (page < 0 || page >= p.num_pages) {
        if (tid % TPR == 0) atomicOr(p.status, JV_STATUS_BAD_PAGE);
      } else {
        const __nv_bfloat16* src = p.cache + ((size_t)page * p.page_size + (j - pi * p.page_size)) * dk;
        __nv_bfloat16* dst = Ks + ((size_t)buf * BLOCK_N + n) * ks;
        for (int c8 = (tid % TPR) * 8; c8 < dk; c8 += TPR * 8) cp_async16(dst + c8, src + c8);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };

  const int r0 = rw * 16 + (lane >> 2), r1 = r0 + 8;       // the two rows this thread holds parts of
  const int pos0 = row_pos_s[r0], pos1 = row_pos_s[r1];
  const bool warp_has_rows = __any_sync(0xffffffffu, pos0 >= 0 || pos1 >= 0);
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[DVW / 8][4];
#pragma unroll
  for (int i = 0; i < DVW / 8; ++i)
#pragma unroll
    for (int k = 0; k < 4; ++k) o[i][k] = 0.f;

  const int n_chunks = (j_hi - j_lo + BLOCK_N - 1) / BLOCK_N;
  load_chunk(j_lo, 0);
  for (int ci = 0; ci < n_chunks; ++ci) {
    const int j0 = j_lo + ci * BLOCK_N, buf = ci & 1;
    if (ci + 1 < n_chunks) {
      load_chunk(j0 + BLOCK_N, buf ^ 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
    const __nv_bfloat16* Kc = Ks + (size_t)buf * BLOCK_N * ks;
    if (!warp_has_rows) {      // none of this warp's 16 rows holds a (token, head): it only helps copying (both warps of a
      __syncthreads();         // row skip alike, so nobody waits at their barrier)
      continue;
    }

    // ---- scores of this warp's 16 rows against the chunk's 32 keys
    // two sets of accumulators take the k steps in turn (eight independent products in flight a warp), added at the
    // end.  Where two warps share a row's output columns (WD == 2) each forms the scores over half of k and the two
    // exchange their partial sums through shared memory: a + b and b + a are the same bits, so both hold the same scores.
    float s[4][4], s2[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int k = 0; k < 4; ++k) s[i][k] = s2[i][k] = 0.f;
    const __nv_bfloat16* qa = Qs + (rw * 16 + (lane & 15)) * qs + (lane >> 4) * 8;
    const __nv_bfloat16* kb = Kc + ((lane & 7) + (lane >> 4) * 8) * ks + ((lane >> 3) & 1) * 8;
    const int khalf = ((dkp / 16 + 1) / 2) * 16;
    const int kbeg = WD == 2 ? dw * khalf : 0, kend = WD == 2 ? min(dkp, kbeg + khalf) : dkp;
    for (int kk = kbeg; kk < kend; kk += 32) {
      uint32_t a[4], b01[4], b23[4];
      ldsm_x4(a, qa + kk);
      ldsm_x4(b01, kb + kk);
      ldsm_x4(b23, kb + 16 * ks + kk);
      mma_bf16(s[0], a, b01[0], b01[1]);
      mma_bf16(s[1], a, b01[2], b01[3]);
      mma_bf16(s[2], a, b23[0], b23[1]);
      mma_bf16(s[3], a, b23[2], b23[3]);
      if (kk + 16 < kend) {
        ldsm_x4(a, qa + kk + 16);
        ldsm_x4(b01, kb + kk + 16);
        ldsm_x4(b23, kb + 16 * ks + kk + 16);
        mma_bf16(s2[0], a, b01[0], b01[1]);
        mma_bf16(s2[1], a, b01[2], b01[3]);
        mma_bf16(s2[2], a, b23[0], b23[1]);
        mma_bf16(s2[3], a, b23[2], b23[3]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int k = 0; k < 4; ++k) s[i][k] += s2[i][k];
    if (WD == 2) {
      // [chunk parity][row warp][column half][16 values][lane]: written here, read by the partner after the pair's barrier;
      // the buffer of this parity is written again two chunks on, after the barrier of the chunk between
      float* mine = Xs + ((((ci & 1) * 4 + rw) * 2 + dw) * 16) * 32 + lane;
      const float* theirs = Xs + ((((ci & 1) * 4 + rw) * 2 + (dw ^ 1)) * 16) * 32 + lane;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) mine[(i * 4 + k) * 32] = s[i][k];
      asm volatile("bar.sync %0, 64;\n" ::"r"(1 + rw) : "memory");
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) s[i][k] += theirs[(i * 4 + k) * 32];
    }
    // ---- mask, running softmax (32-bit)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int j = j0 + i * 8 + (lane & 3) * 2 + (k & 1);
        const int pos = (k < 2) ? pos0 : pos1;
        const bool vis = pos >= 0 && j < j_hi && j <= pos && j >= first_visible(pos, p.window);
        s[i][k] = vis ? s[i][k] * scale_log2 : -INFINITY;
      }
      mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
      mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float al0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - mn0), al1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - mn1);
    m0 = mn0; m1 = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s[i][0] = (mn0 == -INFINITY) ? 0.f : exp2f(s[i][0] - mn0);
      s[i][1] = (mn0 == -INFINITY) ? 0.f : exp2f(s[i][1] - mn0);
      s[i][2] = (mn1 == -INFINITY) ? 0.f : exp2f(s[i][2] - mn1);
      s[i][3] = (mn1 == -INFINITY) ? 0.f : exp2f(s[i][3] - mn1);
      sum0 += s[i][0] + s[i][1];
      sum1 += s[i][2] + s[i][3];
    }
    l0 = l0 * al0 + sum0;     // this thread's share of the row sum; the four threads of a row add up at the end
    l1 = l1 * al1 + sum1;
#pragma unroll
    for (int i = 0; i < DVW / 8; ++i) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }

    // ---- O += P V: P from the registers, V = the chunk's first columns, transposed as it is read
#pragma unroll
    for (int k2 = 0; k2 < 2; ++k2) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * k2][0], s[2 * k2][1]);
      a[1] = pack_bf16(s[2 * k2][2], s[2 * k2][3]);
      a[2] = pack_bf16(s[2 * k2 + 1][0], s[2 * k2 + 1][1]);
      a[3] = pack_bf16(s[2 * k2 + 1][2], s[2 * k2 + 1][3]);
      const __nv_bfloat16* vrow = Kc + (k2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ks + dw * DVW + (lane >> 4) * 8;
#pragma unroll
      for (int i = 0; i < DVW / 16; ++i) {
        uint32_t b[4];
        ldsm_x4_trans(b, vrow + i * 16);
        mma_bf16(o[2 * i], a, b[0], b[1]);
        mma_bf16(o[2 * i + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();       // everybody is done with this buffer before the chunk after next is copied into it
  }

  // ---- row sums over the four threads of a row, then write
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int m = half ? r1 : r0;
    if (row_pos_s[m] < 0) continue;
    const int t = m / p.heads_per_tile, head = hg * p.heads_per_tile + m % p.heads_per_tile;
    const size_t token = (size_t)(q_begin + q_off + t);
    float l = half ? l1 : l0;
    const float mm = half ? m1 : m0;
    float keep = 1.f;
    if (!SPLIT && p.sink != nullptr) {     // the sink joins the denominator, both brought to the larger of the two maxima
      const float sk = p.sink[head] * 1.4426950408889634f, mx = fmaxf(mm, sk);
      keep = (mm == -INFINITY) ? 0.f : exp2f(mm - mx);
      l = l * keep + exp2f(sk - mx);
    }
    size_t slot = 0;
    if (SPLIT) {
      slot = ((size_t)item * p.n_heads + head) * p.n_splits + blockIdx.z;
      if (dw == 0 && (lane & 3) == 0) { p.part_ml[slot * 2] = mm; p.part_ml[slot * 2 + 1] = l; }
    }
    const float inv = keep / l;
#pragma unroll
    for (int i = 0; i < DVW / 8; ++i) {
      const int d = dw * DVW + i * 8 + (lane & 3) * 2;
      const float v0 = o[i][half * 2], v1 = o[i][half * 2 + 1];
      if (SPLIT) {
        if (d < p.dv) p.part_o[slot * p.dv + d] = v0;
        if (d + 1 < p.dv) p.part_o[slot * p.dv + d + 1] = v1;
      } else {
        __nv_bfloat16* dst = p.out + token * p.out_stride + (size_t)head * p.dv;
        if (d < p.dv) dst[d] = __float2bfloat16_rn(v0 * inv);
        if (d + 1 < p.dv) dst[d + 1] = __float2bfloat16_rn(v1 * inv);
      }
    }
  }
}

// Merges the key splits of single-token rows, ascending.  grid = (n_work, n_heads), 128 threads: the splits'
// weights 2^(m_s - m) are formed once into shared memory, then every thread adds up its columns.
constexpr int COMBINE_MAX_SPLITS = 1024;

__global__ void __launch_bounds__(128) latent_combine_kernel(const LatentParams p) {
  __shared__ float w_s[COMBINE_MAX_SPLITS];
  __shared__ float l_s;
  const int x = blockIdx.x, head = blockIdx.y;
  const int entry = p.work[2 * x];
  const int pos = p.start_pos[entry];
  int s_last = pos / p.split_size;
  if (s_last >= p.n_splits) {
    if (threadIdx.x == 0) atomicOr(p.status, JV_STATUS_BAD_ROW);
    s_last = p.n_splits - 1;
  }
  const size_t base = ((size_t)x * p.n_heads + head) * p.n_splits;
  const int s_first = first_visible(pos, p.window) / p.split_size;      // splits before it hold no visible key
  const float sk = p.sink != nullptr ? p.sink[head] * 1.4426950408889634f : -INFINITY;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float m_all = sk;
    for (int s = s_first + lane; s <= s_last; s += 32) m_all = fmaxf(m_all, p.part_ml[(base + s) * 2]);
    m_all = warp_max(m_all);
    float l = 0.f;
    for (int s = s_first + lane; s <= s_last; s += 32) {
      const float w = exp2f(p.part_ml[(base + s) * 2] - m_all);
      w_s[s] = w;
      l += w * p.part_ml[(base + s) * 2 + 1];
    }
    l = warp_sum(l);
    if (p.sink != nullptr) l += exp2f(sk - m_all);      // one more part, with no value
    if (lane == 0) l_s = l;
  }
  __syncthreads();
  const float inv = 1.f / l_s;
  const size_t token = (size_t)p.cu_seqlens[entry];
  __nv_bfloat16* dst = p.out + token * p.out_stride + (size_t)head * p.dv;
  for (int d = threadIdx.x; d < p.dv; d += blockDim.x) {
    float o = 0.f;
    for (int s = s_first; s <= s_last; ++s) o = fmaf(w_s[s], p.part_o[(base + s) * p.dv + d], o);
    dst[d] = __float2bfloat16_rn(o * inv);
  }
}

template <int DVW, int WD>
int launch(const LatentParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
  if (p.n_splits > 0) {
    auto kern = attn_latent_mma_kernel<DVW, WD, true>;
    static size_t allowed = 0;       // set once per size: the attribute call is kept out of stream captures
    if (smem > allowed) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return JV_ERR_UNSUPPORTED;
      allowed = smem;
    }
    kern<<<grid, 128 * WD, smem, stream>>>(p);
    int rc = jv_check_launch();
    if (rc != JV_OK) return rc;
    latent_combine_kernel<<<dim3(grid.x, p.n_heads), 128, 0, stream>>>(p);
    return jv_check_launch();
  }
  auto kern = attn_latent_mma_kernel<DVW, WD, false>;
  static size_t allowed = 0;
  if (smem > allowed) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return JV_ERR_UNSUPPORTED;
    allowed = smem;
  }
  kern<<<grid, 128 * WD, smem, stream>>>(p);
  return jv_check_launch();
}

int out_columns_per_warp(int dv) { return dv <= 32 ? 32 : dv <= 64 ? 64 : dv <= 128 ? 128 : 256; }
}  // namespace

// Rows of a tile that hold tokens: 64 / heads_per_tile, with heads_per_tile = min(heads, 64).
JV_EXPORT int jv_attn_latent_mma_tokens_per_tile(int n_heads) {
  const int hpt = n_heads < BLOCK_M ? n_heads : BLOCK_M;
  return BLOCK_M / hpt;
}

JV_EXPORT int jv_attn_latent_mma_supports(int dk, int dv) {
  if (dk < 8 || (dk % 8) || dv < 1 || dv > dk || dv > 512) return 0;
  const int dkp = (dk + 15) & ~15;
  const int cols = out_columns_per_warp(dv) * (dv > 256 ? 2 : 1);
  const size_t smem = sizeof(__nv_bfloat16) * ((size_t)BLOCK_M * (dkp + PAD) + 2 * (size_t)BLOCK_N * ((dkp > cols ? dkp : cols) + PAD)) +
                      (dv > 256 ? XCH_BYTES : 0);
  return smem <= 220 * 1024;
}

// q: bfloat16 rows of q_stride elements (head h of token n at q[n*q_stride + h*dk]); out: [n, out_stride], head h at
// h*dv; cache: [num_pages, page_size, dk] bfloat16; block_table, cu_seqlens, start_pos, work as for the other paged
// attention kernels; window: the mask (0: causal only); sink: [n_heads] floats or null.  n_splits == 0: every work item attends to all its keys and writes `out`.  n_splits > 0: work
// items are single tokens; part_o [n_work*heads*n_splits*dv] and part_ml [n_work*heads*n_splits*2] floats are scratch.
JV_EXPORT int jv_attn_latent_mma(const void* q, int q_stride, void* out, int out_stride, float* part_o, float* part_ml,
                                 const void* cache, const int* block_table, int table_width, const int* cu_seqlens,
                                 const int* start_pos, const int* work, int n_work, int n_heads, int dk, int dv,
                                 int page_size, int num_pages, float scale, int window, const float* sink, int split_size,
                                 int n_splits, int* status, cudaStream_t stream) {
  if (n_work == 0) return JV_OK;
  if (!jv_attn_latent_mma_supports(dk, dv) || n_heads < 1 || n_splits > COMBINE_MAX_SPLITS || (q_stride % 8) || ((uintptr_t)q % 16) || ((uintptr_t)cache % 16))
    return JV_ERR_UNSUPPORTED;
  LatentParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.part_o = part_o; p.part_ml = part_ml; p.cache = (const __nv_bfloat16*)cache; p.block_table = block_table;
  p.table_width = table_width; p.cu_seqlens = cu_seqlens; p.start_pos = start_pos; p.work = work; p.n_heads = n_heads;
  p.dk = dk; p.dv = dv; p.page_size = page_size; p.num_pages = num_pages; p.scale = scale; p.window = window; p.sink = sink; p.status = status;
  p.heads_per_tile = n_heads < BLOCK_M ? n_heads : BLOCK_M;
  p.tokens_per_tile = n_splits > 0 ? 1 : BLOCK_M / p.heads_per_tile;
  p.split_size = split_size > 0 ? split_size : 1;
  p.n_splits = n_splits;
  const int dkp = (dk + 15) & ~15;
  const int dvw = out_columns_per_warp(dv), wd = dv > 256 ? 2 : 1;
  p.qstride_s = dkp + PAD;
  p.kstride_s = (dkp > dvw * wd ? dkp : dvw * wd) + PAD;
  const size_t smem = sizeof(__nv_bfloat16) * ((size_t)BLOCK_M * p.qstride_s + 2 * (size_t)BLOCK_N * p.kstride_s) +
                      (wd == 2 ? XCH_BYTES : 0);
  dim3 grid(n_work, (n_heads + p.heads_per_tile - 1) / p.heads_per_tile, n_splits > 0 ? n_splits : 1);
  if (wd == 2) return launch<256, 2>(p, grid, smem, stream);
  switch (dvw) {
    case 32: return launch<32, 1>(p, grid, smem, stream);
    case 64: return launch<64, 1>(p, grid, smem, stream);
    case 128: return launch<128, 1>(p, grid, smem, stream);
    default: return launch<256, 1>(p, grid, smem, stream);
  }
}
