// Paged causal attention for bfloat16 on the tensor cores (mma.sync m16n8k16, 32-bit accumulation) for mixers whose
// keys and values differ in size or whose scores are not a plain softmax.  It is the tile code of attn_mma.cu with
// the key size KD and the value size VD as compile-time constants of the LIBRARY (-DJV_KEY_DIM, -DJV_VALUE_DIM:
// one library per pair of sizes that a model needs, built when it is first asked for), and with these options:
//
//   value heads    the value cache is [pages, page, n_v_heads, VD]; key head g reads value head g % n_v_heads
//   score cap      s <- cap * tanh(s / cap) on the scaled score
//   sigmoid        the weight of a visible key is sigmoid(s + bias[query head]); no maximum, no sum, no division
//   float output   two score maps are subtracted by the caller in 32-bit
//   head scale     the scaled score of query head h is multiplied by head_scale[h] (a temperature per head)
//   distance bias  dist_bias[h][min(pos - j, n_dist - 1)] is added to the score of key j; no scale touches it
//   sink           exp(sink[h]) counts once in the softmax's denominator; it has no key and no value
//
// Scores are scaled and masked in 32-bit, the running softmax keeps (max, sum) in 32-bit, weights are rounded to
// bfloat16 for the second product.  Tiles, the split of a decoded token's keys and the merge by the block that ends
// last are those of attn_mma.cu; every wait on a barrier is bounded and reports to the status word.
#include "common.cuh"
#include "mbarrier.cuh"
#include <math.h>

#ifndef JV_KEY_DIM
#define JV_KEY_DIM 64
#endif
#ifndef JV_VALUE_DIM
#define JV_VALUE_DIM 64
#endif

namespace {
constexpr int KD = JV_KEY_DIM, VD = JV_VALUE_DIM;
static_assert(KD % 16 == 0 && VD % 16 == 0 && KD >= 16 && VD >= 16 && KD <= 256 && VD <= 256, "sizes in steps of 16");

constexpr int BN = 64;         // keys per tile
constexpr int NWARPS = 4;
constexpr int THREADS = NWARPS * 32;
constexpr int ROWS_PREFILL = 16 * NWARPS;
constexpr int DECODE_STAGES = 3;
constexpr float LOG2E = 1.4426950408889634f;

struct Params {
  const __nv_bfloat16* q; int q_stride;
  void* out; int out_stride;
  float* part_o; float* part_ml;
  const __nv_bfloat16* k_cache; const __nv_bfloat16* v_cache;
  const int* block_table; int table_width;
  const int* cu_seqlens; const int* start_pos;
  const int* work;
  int n_q_heads, n_kv_heads, page_size, num_pages, window;
  float scale;                 // multiplies q.k
  float score_cap;             // > 0: s <- cap * tanh(s / cap)
  int sigmoid;                 // independent weights sigmoid(s + bias[query head])
  const float* bias;           // [n_q_heads] or null
  const float* head_scale;     // [n_q_heads] or null
  const float* dist_bias;      // [n_q_heads][n_dist] or null: row h serves head h, column = how far back the key lies
  int n_dist;                  //   (distances of n_dist - 1 and more share the last column)
  const float* sink;           // [n_q_heads] or null (softmax only)
  int out_f32;                 // `out` is float
  int n_v_heads;
  int tokens_per_tile, heads_per_tile, n_head_groups, split_size, n_splits;
  int* status;
  int* counters;               // decode: one per (work item, kv head, head group), zero between launches
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // 0 bytes read: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Rows of a shared-memory tile are D elements plus 8 of padding: the row stride in 4-byte words
// is then 4 modulo 8, so the eight 16-byte rows that one ldmatrix phase reads fall into distinct banks.
template <int D> struct Tile { static constexpr int STRIDE = D + 8; };

// Cache slots (page * page_size + place in the page) of keys [j0, j0 + BN) (-1: beyond j_end, or no
// page), one per thread n < BN: the block table is read once per key, ahead of the copies.
__device__ __forceinline__ void tile_rows(long long* rows, const Params& p, int entry, int kv_head, int j0, int j_end,
                                          int tid) {
  if (tid < BN) {
    const int j = j0 + tid;
    long long off = -1;
    if (j < j_end) {
      const int pi = j / p.page_size;
      const int page = pi < p.table_width ? p.block_table[(size_t)entry * p.table_width + pi] : -1;
      if (page < 0 || page >= p.num_pages) atomicOr(p.status, JV_STATUS_BAD_PAGE);
      else off = (long long)page * p.page_size + (j - pi * p.page_size);
    }
    rows[tid] = off;
  }
}

// ---- mbarrier + bulk-copy (TMA) helpers.  A cache row of one kv head is D contiguous elements, so a
// 64-key tile is 64 + 64 bulk copies, one per thread, instead of 16-byte copies by the thousand; their
// completion is counted in bytes on the stage's mbarrier.
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, int bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Copies the rows listed by tile_rows into a K tile and a V tile: thread n < 64 the key row n, thread
// 64 + n the value row n (a row without a source is zeroed by the thread).  Every thread arrives once
// on `bar`, which completes when all bytes have landed.
__device__ __forceinline__ void issue_tile(__nv_bfloat16* ks, __nv_bfloat16* vs, const long long* rows, const Params& p,
                                           int kv_head, uint64_t* bar, int tid) {
  static_assert(THREADS == 2 * BN, "one thread per key row and per value row");
  const int n = tid & (BN - 1);
  const bool is_v = tid >= BN;
  const long long slot = rows[n];
  const int dim = is_v ? VD : KD;
  __nv_bfloat16* dst = is_v ? vs + n * Tile<VD>::STRIDE : ks + n * Tile<KD>::STRIDE;
  if (slot >= 0) {
    const __nv_bfloat16* src = is_v ? p.v_cache + (slot * p.n_v_heads + kv_head % p.n_v_heads) * VD
                                    : p.k_cache + (slot * p.n_kv_heads + kv_head) * KD;
    mbar_expect_tx(bar, dim * 2);
    bulk_copy(dst, src, dim * 2, bar);
  } else {
    for (int c = 0; c < dim / 8; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
    mbar_arrive(bar);
  }
}

// Waits for a tile; on a timeout records it in the status word (the caller then leaves).
__device__ __forceinline__ bool wait_tile(uint64_t* bar, int parity, const Params& p) {
  if (mbar_wait(bar, parity)) return true;
  atomicOr(p.status, JV_STATUS_WAIT_EXPIRED);
  return false;
}

// S[16 rows, NB*8 keys] += Q[16, D] K[keys, D]^T for one warp.  `qs` points at the warp's first
// row, `ks` at the first key row.
template <int D, int NB>
__device__ __forceinline__ void qk_tile(float (&s)[NB][4], const __nv_bfloat16* qs, const __nv_bfloat16* ks, int lane) {
  constexpr int S = Tile<D>::STRIDE;
  const int mat = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[4];
    ldmatrix_x4(a, qs + ((mat & 1) * 8 + r) * S + kk * 16 + (mat >> 1) * 8);
#pragma unroll
    for (int nb2 = 0; nb2 < NB / 2; ++nb2) {
      uint32_t b[4];
      ldmatrix_x4(b, ks + (nb2 * 16 + (mat >> 1) * 8 + r) * S + kk * 16 + (mat & 1) * 8);
      mma_bf16(s[2 * nb2], a, b[0], b[1]);
      mma_bf16(s[2 * nb2 + 1], a, b[2], b[3]);
    }
  }
}

// O[16, D] += P[16, NB*8 keys] V[keys, D] for one warp; P comes from the score registers.
template <int D, int NB>
__device__ __forceinline__ void pv_tile(float (&o)[D / 8][4], const float (&pr)[NB][4], const __nv_bfloat16* vs, int lane) {
  constexpr int S = Tile<D>::STRIDE;
  const int mat = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kk = 0; kk < NB / 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(pr[2 * kk][0], pr[2 * kk][1]);
    a[1] = pack_bf16(pr[2 * kk][2], pr[2 * kk][3]);
    a[2] = pack_bf16(pr[2 * kk + 1][0], pr[2 * kk + 1][1]);
    a[3] = pack_bf16(pr[2 * kk + 1][2], pr[2 * kk + 1][3]);
#pragma unroll
    for (int db2 = 0; db2 < D / 16; ++db2) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, vs + (kk * 16 + (mat & 1) * 8 + r) * S + db2 * 16 + (mat >> 1) * 8);
      mma_bf16(o[2 * db2], a, b[0], b[1]);
      mma_bf16(o[2 * db2 + 1], a, b[2], b[3]);
    }
  }
}

// 1 / x to about 2^-23 relative (1 / inf = 0), one instruction instead of the dozen of an IEEE division
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// Turns one warp's raw products of a tile into weights.  The products are scaled (and capped) first.  Softmax:
// exponentials against the running maximum of the thread's two rows, (max, sum) updated, output accumulators
// rescaled.  Sigmoid: every weight stands alone, nothing is kept.  With MASK the visibility test is applied
// (key0 + nb*8 + (lane%4)*2 + (i&1) is the key of s[nb][i]; pos0/pos1 are the positions of rows lane/4 and
// lane/4 + 8, -1 for an unused row); tiles that lie wholly inside every row's visible range go without it.
template <int NB, bool MASK>
__device__ __forceinline__ void weights_tile(float (&s)[NB][4], float (&o)[VD / 8][4], float (&m)[2], float (&l)[2],
                                             int pos0, int pos1, int key0, int j_end, int window, float scale0,
                                             float scale1, const float* dist0, const float* dist1, int n_dist,
                                             float cap, bool sigmoid, float bias0, float bias1, int lane) {
  const float cap_exp = cap > 0.f ? 2.f * LOG2E / cap : 0.f;
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v = s[nb][i] * ((i < 2) ? scale0 : scale1);
      if (dist0 != nullptr) {     // by how far back the key lies; rows without a position and hidden keys read column 0
        const int back = ((i < 2) ? pos0 : pos1) - (key0 + nb * 8 + (lane & 3) * 2 + (i & 1));
        v += __ldg(((i < 2) ? dist0 : dist1) + min(max(back, 0), n_dist - 1));
      }
      // tanh(x) = 1 - 2 / (1 + e^(2x)): one ex2 and one reciprocal; its absolute error (about 1e-7) times the cap is
      // far below what the 16-bit operands of the product leave in a score
      if (cap > 0.f) v = fmaf(-2.f * cap, fast_rcp(1.f + fast_exp2(v * cap_exp)), cap);
      s[nb][i] = v;
    }
  if (sigmoid) {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        bool vis = true;
        if (MASK) {
          const int key = key0 + nb * 8 + (lane & 3) * 2 + (i & 1);
          const int pos = (i < 2) ? pos0 : pos1;
          vis = key < j_end && key <= pos && key >= first_visible(pos, window);
        }
        const float x = s[nb][i] + ((i < 2) ? bias0 : bias1);
        s[nb][i] = vis ? fast_rcp(1.f + fast_exp2(-x * LOG2E)) : 0.f;
      }
    return;
  }
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (MASK) {
        const int key = key0 + nb * 8 + (lane & 3) * 2 + (i & 1);
        const int pos = (i < 2) ? pos0 : pos1;
        const bool vis = key < j_end && key <= pos && key >= first_visible(pos, window);
        if (!vis) s[nb][i] = -INFINITY;
      }
      mx[i >> 1] = fmaxf(mx[i >> 1], s[nb][i]);
    }
  float alpha[2], m_scaled[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    const float m_new = fmaxf(m[h], mx[h]);
    alpha[h] = (m[h] == -INFINITY) ? 0.f : fast_exp2((m[h] - m_new) * LOG2E);  // m_new == -inf only if m[h] is
    m_scaled[h] = (m_new == -INFINITY) ? 0.f : m_new * LOG2E;                   // then every score is -inf: p = 0
    m[h] = m_new;
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float pr = fast_exp2(fmaf(s[nb][i], LOG2E, -m_scaled[i >> 1]));
      s[nb][i] = pr;
      sum[i >> 1] += pr;
    }
#pragma unroll
  for (int h = 0; h < 2; ++h) l[h] = l[h] * alpha[h] + sum[h];   // per-thread part; lanes are summed at the end
  if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
    for (int db = 0; db < VD / 8; ++db) {
      o[db][0] *= alpha[0]; o[db][1] *= alpha[0];
      o[db][2] *= alpha[1]; o[db][3] *= alpha[1];
    }
  }
}

// ------------------------------------------------------------------------- prefill
__global__ void __launch_bounds__(THREADS) attn_prefill_general_kernel(const Params p) {
  constexpr int SK = Tile<KD>::STRIDE, SV = Tile<VD>::STRIDE;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);    // [64][SK]
  __nv_bfloat16* ks = qs + ROWS_PREFILL * SK;                         // [2][BN][SK]
  __nv_bfloat16* vs = ks + 2 * BN * SK;                               // [2][BN][SV]
  __shared__ long long rows[2][BN];
  __shared__ __align__(8) uint64_t bars[2];
  pdl_trigger();
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], THREADS);
    mbar_init(&bars[1], THREADS);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  pdl_wait();

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // the work list is in ascending order of a tile's first token: taken from its end, the tiles with the most keys
  // start first and the short ones fill the last wave
  const int item = gridDim.x - 1 - blockIdx.x;
  const int entry = p.work[2 * item], q_off = p.work[2 * item + 1];
  const int kv_head = blockIdx.y / p.n_head_groups, hg = blockIdx.y % p.n_head_groups;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int HPT = p.heads_per_tile;
  const int q_begin = p.cu_seqlens[entry];
  const int q_len = p.cu_seqlens[entry + 1] - q_begin;
  const int ctx = p.start_pos[entry];
  const int tokens_here = min(p.tokens_per_tile, q_len - q_off);
  if (tokens_here <= 0) return;
  const int pos_first = ctx + q_off;
  const int j_lo = first_visible(pos_first, p.window);
  const int j_hi = pos_first + tokens_here;   // exclusive

  // ---- queries of the tile (unused rows zero)
  constexpr int CH = KD / 8;
  for (int c = tid; c < ROWS_PREFILL * CH; c += THREADS) {
    const int r = c / CH, part = c - r * CH;
    const int t = r / HPT, hh = hg * HPT + r % HPT;
    const bool valid = t < tokens_here && hh < G;
    const size_t off = valid ? (size_t)(q_begin + q_off + t) * p.q_stride + (size_t)(kv_head * G + hh) * KD + part * 8 : 0;
    cp_async16(qs + r * SK + part * 8, p.q + off, valid);
  }
  const int n_tiles = (j_hi - j_lo + BN - 1) / BN;
  tile_rows(rows[0], p, entry, kv_head, j_lo, j_hi, tid);
  tile_rows(rows[1], p, entry, kv_head, j_lo + BN, j_hi, tid);
  cp_async_commit();                      // the queries
  __syncthreads();
  issue_tile(ks, vs, rows[0], p, kv_head, &bars[0], tid);
  __syncthreads();                        // rows[0] has been read by all before iteration 0 refills it

  // ---- this thread's two rows
  int pos[2], row_head[2];
  float bias[2] = {0.f, 0.f};
  {
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
    const int t0 = r0 / HPT, h0 = hg * HPT + r0 % HPT, t1 = r1 / HPT, h1 = hg * HPT + r1 % HPT;
    pos[0] = (t0 < tokens_here && h0 < G) ? pos_first + t0 : -1;
    pos[1] = (t1 < tokens_here && h1 < G) ? pos_first + t1 : -1;
    if (p.bias != nullptr) {
      if (h0 < G) bias[0] = p.bias[kv_head * G + h0];
      if (h1 < G) bias[1] = p.bias[kv_head * G + h1];
    }
    row_head[0] = kv_head * G + min(h0, G - 1);
    row_head[1] = kv_head * G + min(h1, G - 1);
  }
  float scale[2] = {p.scale, p.scale};
  const float* dist[2] = {nullptr, nullptr};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (p.head_scale != nullptr) scale[h] *= p.head_scale[row_head[h]];
    if (p.dist_bias != nullptr) dist[h] = p.dist_bias + (size_t)row_head[h] * p.n_dist;
  }
  const bool sigmoid = p.sigmoid != 0;
  // the last position any row of this warp has (its tiles beyond that are skipped)
  int warp_last = max(pos[0], pos[1]);
  int warp_first = min(pos[0] < 0 ? 0x7fffffff : pos[0], pos[1] < 0 ? 0x7fffffff : pos[1]);   // over rows in use
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    warp_last = max(warp_last, __shfl_xor_sync(0xffffffffu, warp_last, o));
    warp_first = min(warp_first, __shfl_xor_sync(0xffffffffu, warp_first, o));
  }

  float o_acc[VD / 8][4];
#pragma unroll
  for (int db = 0; db < VD / 8; ++db)
#pragma unroll
    for (int i = 0; i < 4; ++i) o_acc[db][i] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < n_tiles)
      issue_tile(ks + (buf ^ 1) * BN * SK, vs + (buf ^ 1) * BN * SV, rows[buf ^ 1], p, kv_head, &bars[buf ^ 1], tid);
    // rows of tile t+2 go where those of tile t were (read when tile t was issued, an iteration ago)
    if (t + 2 < n_tiles) tile_rows(rows[buf], p, entry, kv_head, j_lo + (t + 2) * BN, j_hi, tid);
    if (t == 0) cp_async_wait<0>();
    // every thread takes the same way out: all saw the tile, or the block stops (status word set)
    if (!__syncthreads_and(wait_tile(&bars[buf], (t >> 1) & 1, p))) {
      wait_tile(&bars[buf], (t >> 1) & 1, p);   // once more, bounded, for copies that may still be landing
      return;
    }
    const int key0 = j_lo + t * BN;
    if (key0 <= warp_last) {
      float s[BN / 8][4];
#pragma unroll
      for (int nb = 0; nb < BN / 8; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[nb][i] = 0.f;
      qk_tile<KD, BN / 8>(s, qs + warp * 16 * SK, ks + buf * BN * SK, lane);
      // the test is needed only where the tile reaches past the first row's position, past the end,
      // or a window cuts into it
      if (key0 + BN - 1 > warp_first || key0 + BN > j_hi || p.window != 0)
        weights_tile<BN / 8, true>(s, o_acc, m, l, pos[0], pos[1], key0, j_hi, p.window, scale[0], scale[1], dist[0], dist[1], p.n_dist, p.score_cap, sigmoid,
                                   bias[0], bias[1], lane);
      else
        weights_tile<BN / 8, false>(s, o_acc, m, l, pos[0], pos[1], key0, j_hi, p.window, scale[0], scale[1], dist[0], dist[1], p.n_dist, p.score_cap, sigmoid,
                                    bias[0], bias[1], lane);
      pv_tile<VD, BN / 8>(o_acc, s, vs + buf * BN * SV, lane);
    }
    __syncthreads();
  }

  // ---- normalise and write
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (pos[h] < 0) continue;
    const int r = warp * 16 + (lane >> 2) + h * 8;
    const int t = r / HPT, hh = hg * HPT + r % HPT;
    const size_t at = (size_t)(q_begin + q_off + t) * p.out_stride + (size_t)(kv_head * G + hh) * VD;
    float inv = sigmoid ? 1.f : 1.f / l[h];
    if (p.sink != nullptr) {     // the sink joins the denominator, both brought to the larger of the two maxima
      const float sk = p.sink[row_head[h]], mx = fmaxf(m[h], sk);
      const float e = __expf(m[h] - mx);
      inv = e / (l[h] * e + __expf(sk - mx));
    }
#pragma unroll
    for (int db = 0; db < VD / 8; ++db) {
      const int d = db * 8 + (lane & 3) * 2;
      if (p.out_f32)
        *reinterpret_cast<float2*>((float*)p.out + at + d) = make_float2(o_acc[db][2 * h] * inv, o_acc[db][2 * h + 1] * inv);
      else
        *reinterpret_cast<uint32_t*>((__nv_bfloat16*)p.out + at + d) = pack_bf16(o_acc[db][2 * h] * inv, o_acc[db][2 * h + 1] * inv);
    }
  }
}

// -------------------------------------------------------------------------- decode
__global__ void __launch_bounds__(THREADS) attn_decode_general_kernel(const Params p) {
  constexpr int SK = Tile<KD>::STRIDE, SV = Tile<VD>::STRIDE;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);    // [16][SK]
  __nv_bfloat16* ks = qs + 16 * SK;                                   // [STAGES][BN][SK]
  __nv_bfloat16* vs = ks + DECODE_STAGES * BN * SK;                   // [STAGES][BN][SV]
  __shared__ long long rows[DECODE_STAGES][BN];
  __shared__ int is_last;
  __shared__ __align__(8) uint64_t bars[DECODE_STAGES];
  pdl_trigger();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int st = 0; st < DECODE_STAGES; ++st) mbar_init(&bars[st], THREADS);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  pdl_wait();

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int entry = p.work[2 * blockIdx.x];
  const int kv_head = blockIdx.y / p.n_head_groups, hg = blockIdx.y % p.n_head_groups;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int HPT = p.heads_per_tile;
  const int pos_q = p.start_pos[entry];
  const int vis_lo = first_visible(pos_q, p.window);   // visible keys: [vis_lo, pos_q]
  const int j_lo = max(vis_lo, (int)blockIdx.z * p.split_size);
  const int j_hi = min(pos_q + 1, ((int)blockIdx.z + 1) * p.split_size);
  if (j_lo >= j_hi) return;
  const int token = p.cu_seqlens[entry];

  constexpr int CH = KD / 8;
  for (int c = tid; c < 16 * CH; c += THREADS) {
    const int r = c / CH, part = c - r * CH;
    const int hh = hg * HPT + r;
    const bool valid = r < HPT && hh < G;
    const size_t off = valid ? (size_t)token * p.q_stride + (size_t)(kv_head * G + hh) * KD + part * 8 : 0;
    cp_async16(qs + r * SK + part * 8, p.q + off, valid);
  }
  const int n_tiles = (j_hi - j_lo + BN - 1) / BN;
#pragma unroll
  for (int st = 0; st < DECODE_STAGES; ++st) tile_rows(rows[st], p, entry, kv_head, j_lo + st * BN, j_hi, tid);
  cp_async_commit();                      // the queries
  __syncthreads();
#pragma unroll
  for (int st = 0; st < DECODE_STAGES - 1; ++st)
    if (st < n_tiles) issue_tile(ks + st * BN * SK, vs + st * BN * SV, rows[st], p, kv_head, &bars[st], tid);
  __syncthreads();                        // rows[0] has been read by all before iteration 0 refills it

  // every row is the same token: position pos_q for rows that hold a head, -1 otherwise
  int pos[2], row_head[2];
  float bias[2] = {0.f, 0.f};
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
    pos[0] = (r0 < HPT && hg * HPT + r0 < G) ? pos_q : -1;
    pos[1] = (r1 < HPT && hg * HPT + r1 < G) ? pos_q : -1;
    if (p.bias != nullptr) {
      if (pos[0] >= 0) bias[0] = p.bias[kv_head * G + hg * HPT + r0];
      if (pos[1] >= 0) bias[1] = p.bias[kv_head * G + hg * HPT + r1];
    }
    row_head[0] = kv_head * G + min(hg * HPT + r0, G - 1);
    row_head[1] = kv_head * G + min(hg * HPT + r1, G - 1);
  }
  float scale[2] = {p.scale, p.scale};
  const float* dist[2] = {nullptr, nullptr};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (p.head_scale != nullptr) scale[h] *= p.head_scale[row_head[h]];
    if (p.dist_bias != nullptr) dist[h] = p.dist_bias + (size_t)row_head[h] * p.n_dist;
  }
  const bool sigmoid = p.sigmoid != 0;
  float o_acc[VD / 8][4];
#pragma unroll
  for (int db = 0; db < VD / 8; ++db)
#pragma unroll
    for (int i = 0; i < 4; ++i) o_acc[db][i] = 0.f;
  // sigmoid weights are sums without a maximum: every part is merged with the factor exp2(0 - 0) = 1
  float m[2] = {sigmoid ? 0.f : -INFINITY, sigmoid ? 0.f : -INFINITY}, l[2] = {0.f, 0.f};

  for (int t = 0; t < n_tiles; ++t) {
    const int nxt = t + DECODE_STAGES - 1;
    if (nxt < n_tiles) {
      const int nb = nxt % DECODE_STAGES;
      issue_tile(ks + nb * BN * SK, vs + nb * BN * SV, rows[nb], p, kv_head, &bars[nb], tid);
    }
    // rows of tile t+STAGES go where those of tile t were (read when tile t was issued)
    if (t + DECODE_STAGES < n_tiles)
      tile_rows(rows[t % DECODE_STAGES], p, entry, kv_head, j_lo + (t + DECODE_STAGES) * BN, j_hi, tid);
    if (t == 0) cp_async_wait<0>();
    if (!__syncthreads_and(wait_tile(&bars[t % DECODE_STAGES], (t / DECODE_STAGES) & 1, p))) {
      wait_tile(&bars[t % DECODE_STAGES], (t / DECODE_STAGES) & 1, p);
      return;
    }
    const int buf = t % DECODE_STAGES;
    const int key0 = j_lo + t * BN + warp * 16;      // this warp's 16 keys of the tile
    if (key0 < j_hi) {
      float s[2][4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[nb][i] = 0.f;
      qk_tile<KD, 2>(s, qs, ks + (buf * BN + warp * 16) * SK, lane);
      // keys before j_lo are never loaded, so only the tile that reaches past j_hi needs the test
      if (key0 + 16 > j_hi)
        weights_tile<2, true>(s, o_acc, m, l, pos[0], pos[1], key0, j_hi, 0, scale[0], scale[1], dist[0], dist[1], p.n_dist, p.score_cap, sigmoid, bias[0], bias[1], lane);
      else
        weights_tile<2, false>(s, o_acc, m, l, pos[0], pos[1], key0, j_hi, 0, scale[0], scale[1], dist[0], dist[1], p.n_dist, p.score_cap, sigmoid, bias[0], bias[1], lane);
      pv_tile<VD, 2>(o_acc, s, vs + (buf * BN + warp * 16) * SV, lane);
    }
    __syncthreads();
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    m[h] *= LOG2E;          // from here on the maxima are exponents of two (warps and splits are merged with exp2)
  }

  // ---- merge the four warps (each saw a quarter of the keys) through shared memory
  constexpr int D = VD;
  float* mo = reinterpret_cast<float*>(ks);            // [NWARPS][16][VD]  (the tiles are done with)
  float* mm = mo + NWARPS * 16 * D;                    // [NWARPS][16]
  float* ml = mm + NWARPS * 16;                        // [NWARPS][16]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = (lane >> 2) + h * 8;
    if (r >= HPT) continue;               // rows without a head are not merged
    if ((lane & 3) == 0) { mm[warp * 16 + r] = m[h]; ml[warp * 16 + r] = l[h]; }
#pragma unroll
    for (int db = 0; db < D / 8; ++db) {
      const int d = db * 8 + (lane & 3) * 2;
      mo[(warp * 16 + r) * D + d] = o_acc[db][2 * h];
      mo[(warp * 16 + r) * D + d + 1] = o_acc[db][2 * h + 1];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < HPT * D; idx += THREADS) {
    const int r = idx / D, d = idx - r * D;
    const int hh = hg * HPT + r;
    if (hh >= G) continue;
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) m_all = fmaxf(m_all, mm[w * 16 + r]);
    float o = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      const float mw = mm[w * 16 + r];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m_all);
      o += f * mo[(w * 16 + r) * D + d];
      lsum += f * ml[w * 16 + r];
    }
    const size_t slot = ((size_t)blockIdx.x * p.n_q_heads + (kv_head * G + hh)) * p.n_splits + blockIdx.z;
    p.part_o[slot * D + d] = o;
    if (d == 0) { p.part_ml[slot * 2] = m_all; p.part_ml[slot * 2 + 1] = lsum; }
  }

  // ---- the block that finishes last among the splits of this (token, kv head, head group) merges them,
  //      in ascending order of the splits whichever block that is.  Nobody waits: a block adds one to the
  //      counter when its partial result is written and leaves unless it brought the count to the total.
  const int s_first = vis_lo / p.split_size;
  int s_last = pos_q / p.split_size;
  if (s_last >= p.n_splits) {           // the launch has too few splits for this length
    if (tid == 0) atomicOr(p.status, JV_STATUS_BAD_ROW);
    s_last = p.n_splits - 1;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int* counter = p.counters + (size_t)blockIdx.x * gridDim.y + blockIdx.y;
    const int done = atomicAdd(counter, 1) + 1;
    is_last = (done == s_last - s_first + 1);
    if (is_last) *counter = 0;          // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int idx = tid; idx < HPT * D; idx += THREADS) {
    const int r = idx / D, d = idx - r * D;
    const int hh = hg * HPT + r;
    if (hh >= G) continue;
    const int head = kv_head * G + hh;
    const size_t base = ((size_t)blockIdx.x * p.n_q_heads + head) * p.n_splits;
    // the sink is one more part, with no value: maximum sink, sum 1 (maxima are exponents of two here)
    const float sk = p.sink != nullptr ? p.sink[head] * LOG2E : -INFINITY;
    float m_all = sk;
    for (int sp = s_first; sp <= s_last; ++sp) m_all = fmaxf(m_all, __ldcg(p.part_ml + (base + sp) * 2));
    float o = 0.f, l_all = p.sink != nullptr ? exp2f(sk - m_all) : 0.f;
    for (int sp = s_first; sp <= s_last; ++sp) {
      const float f = exp2f(__ldcg(p.part_ml + (base + sp) * 2) - m_all);
      l_all += f * __ldcg(p.part_ml + (base + sp) * 2 + 1);
      o += f * __ldcg(p.part_o + (base + sp) * D + d);
    }
    const float res = sigmoid ? o : o / l_all;
    if (p.out_f32) ((float*)p.out)[(size_t)token * p.out_stride + (size_t)head * D + d] = res;
    else ((__nv_bfloat16*)p.out)[(size_t)token * p.out_stride + (size_t)head * D + d] = __float2bfloat16_rn(res);
  }
}

size_t prefill_smem() {
  return sizeof(__nv_bfloat16) * ((size_t)(ROWS_PREFILL + 2 * BN) * Tile<KD>::STRIDE + (size_t)2 * BN * Tile<VD>::STRIDE);
}
size_t decode_smem() {
  const size_t q = sizeof(__nv_bfloat16) * 16 * Tile<KD>::STRIDE;
  const size_t tiles = sizeof(__nv_bfloat16) * (size_t)DECODE_STAGES * BN * (Tile<KD>::STRIDE + Tile<VD>::STRIDE);
  const size_t merge = sizeof(float) * (NWARPS * 16 * VD + 2 * NWARPS * 16);
  return q + (tiles > merge ? tiles : merge);
}

int launch(const Params& p, int n_work, bool split, cudaStream_t stream) {
  if (!split) {
    static bool ready[JV_MAX_DEVICES];
    const size_t smem = prefill_smem();
    if (!jv_once_per_device(ready, [&] {
          return cudaFuncSetAttribute(attn_prefill_general_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
        }))
      return JV_ERR_UNSUPPORTED;
    dim3 grid(n_work, p.n_kv_heads * p.n_head_groups);
    return jv_launch(attn_prefill_general_kernel, grid, dim3(THREADS), smem, stream, p);
  }
  static bool ready[JV_MAX_DEVICES];
  const size_t smem = decode_smem();
  if (!jv_once_per_device(ready, [&] {
        return cudaFuncSetAttribute(attn_decode_general_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
      }))
    return JV_ERR_UNSUPPORTED;
  dim3 grid(n_work, p.n_kv_heads * p.n_head_groups, p.n_splits);
  return jv_launch(attn_decode_general_kernel, grid, dim3(THREADS), smem, stream, p);
}
}  // namespace

// The sizes this library was built for.
JV_EXPORT int jv_attn_general_key_dim() { return KD; }
JV_EXPORT int jv_attn_general_value_dim() { return VD; }

// Tokens in a prefill tile: 64 rows / heads per tile, heads per tile = min(G, 16).
JV_EXPORT int jv_attn_general_tokens_per_tile(int n_q_heads, int n_kv_heads) {
  const int G = n_q_heads / n_kv_heads;
  return ROWS_PREFILL / (G < 16 ? G : 16);
}

// Arguments as for jv_attn_simt_ex (csrc/attn_simt.cu), bfloat16 only, for the key and value sizes of this library.
// v_cache: [num_pages, page_size, n_v_heads, VD].  n_splits == 0: prompt portions, work = (entry, first token of the
// tile).  n_splits > 0: single tokens, part_o [n_work*Hq*n_splits*VD] and part_ml [n_work*Hq*n_splits*2] floats of
// scratch, and `counters`, n_work * n_kv_heads * ceil(G/16) ints that are zero before the launch (the kernel leaves
// them zero).
JV_EXPORT int jv_attn_general_mma(const void* q, int q_stride, void* out, int out_stride, int out_f32, float* part_o,
                                  float* part_ml, int* counters, const void* k_cache, const void* v_cache,
                                  const int* block_table, int table_width, const int* cu_seqlens, const int* start_pos,
                                  const int* work, int n_work, int n_q_heads, int n_kv_heads, int n_v_heads, int key_dim,
                                  int value_dim, int page_size, int num_pages, int window, float scale, float score_cap,
                                  int sigmoid, const float* bias, const float* head_scale, const float* dist_bias,
                                  int n_dist, const float* sink, int split_size, int n_splits, int* status,
                                  cudaStream_t stream) {
  if (n_work == 0) return JV_OK;
  if ((dist_bias != nullptr && n_dist < 1) || (sink != nullptr && sigmoid)) return JV_ERR_UNSUPPORTED;
  if (key_dim != KD || value_dim != VD || n_kv_heads < 1 || n_v_heads < 1 || n_q_heads % n_kv_heads != 0)
    return JV_ERR_UNSUPPORTED;
  if ((q_stride % 8) || (out_stride % 2) || ((uintptr_t)q % 16) || ((uintptr_t)out % 8) || ((uintptr_t)k_cache % 16) ||
      ((uintptr_t)v_cache % 16))
    return JV_ERR_UNSUPPORTED;   // 16-byte copies need aligned rows
  if (prefill_smem() > 227 * 1024 || decode_smem() > 227 * 1024) return JV_ERR_UNSUPPORTED;
  Params p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.out = out; p.out_stride = out_stride; p.out_f32 = out_f32 ? 1 : 0;
  p.part_o = part_o; p.part_ml = part_ml; p.counters = counters;
  p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
  p.block_table = block_table; p.table_width = table_width; p.cu_seqlens = cu_seqlens; p.start_pos = start_pos;
  p.work = work; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.n_v_heads = n_v_heads; p.page_size = page_size;
  p.num_pages = num_pages; p.window = window; p.scale = scale; p.score_cap = score_cap; p.sigmoid = sigmoid ? 1 : 0;
  p.bias = bias; p.status = status;
  p.head_scale = head_scale; p.dist_bias = dist_bias; p.n_dist = n_dist; p.sink = sink;
  const int G = n_q_heads / n_kv_heads;
  p.heads_per_tile = G < 16 ? G : 16;
  p.n_head_groups = (G + p.heads_per_tile - 1) / p.heads_per_tile;
  p.tokens_per_tile = n_splits > 0 ? 1 : ROWS_PREFILL / p.heads_per_tile;
  p.split_size = split_size > 0 ? split_size : 1;
  p.n_splits = n_splits;
  return launch(p, n_work, n_splits > 0, stream);
}
