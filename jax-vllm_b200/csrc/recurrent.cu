// Mixers whose memory is a matrix per head that is carried from token to token (a fixed-size state per request
// instead of keys and values per token).  Everything that enters the recurrence is 32-bit: the state, decays,
// gates, unit keys, the running maximum; the projections that feed it may be 16-bit.
//
// Both recurrences built here are cases of ONE update of a state S [key channel, value channel] per head,
//
//     S <- diag(w_t) S - b_t (u_t^T S) + k_t v_t^T          (both terms read the old S)
//     o_t = S^T r_t                                          (the new S)
//
// so they share the scan kernel and differ in the kernel that prepares (r, k, w, u, b) per token and head:
//
//   generalized delta rule   w = exp(-e^(-1/2) sigmoid(z_w + w0)), a = sigmoid(z_a + a0), u = k / sqrt(|k|^2 + 1e-6),
//                            b = a * u                                              (jv_delta_prepare, per token)
//   matrix memory with exponential gates and a running maximum m (m starts at 0):
//                            i = cap tanh((z_i + i0) / cap), f = logsigmoid(cap tanh((z_f + f0) / cap)),
//                            m' = max(f + m, i), keep = exp(f + m - m'), take = exp(i - m'),
//                            n <- keep n + take k, den = max(|n . q|, exp(-m')) + 1e-6,
//                            w = keep (every channel), k <- take k, r = q, no removal term; n is one more column
//                            of the state whose value is 1, so n . q is that column's output, and o is divided by
//                            den when the heads are normed          (jv_memory_gates: a scan over m alone, one warp a
//                                                                    head, an add and a max a token; then all tokens
//                                                                    at once)
//
// The columns of S evolve independently of one another, so the scan is parallel over (entry, head, value column) and
// serial over an entry's tokens: a warp holds 8 columns x 4 lanes that share the key channels; a thread keeps its
// KPT = ceil(key size / 4) state elements in registers from the entry's first token to its last, the per-token
// vectors pass through shared memory in chunks that are fetched (cp.async) while the chunk before is computed, and
// the two dot products of a token are two shuffles each.  A step of single tokens is the same kernel with one token
// an entry: it then reads and writes the state once, which is all its traffic.
//
// jv_head_norm_gate finishes both: each head's output divided by its root mean square, times a weight per element,
// times sigmoid(gate), rounded for the output product.
#include "common.cuh"
#include <math.h>

namespace {

// ---------------------------------------------------------------------------------------------------- prepare
// packed: [n, heads, NV, D] float, vectors in the order r, k, w, u, b.
template <typename T, typename W>
__global__ void __launch_bounds__(128) delta_prepare_kernel(const T* __restrict__ proj, long long stride, int r_off,
                                                            int k_off, int a_off, const T* __restrict__ zw,
                                                            long long zw_stride, const W* __restrict__ a_bias,
                                                            const W* __restrict__ w_bias, float* __restrict__ packed,
                                                            int heads, int D) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x, h = blockIdx.y;
  const T* row = proj + (size_t)n * stride;
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float k = to_f32(row[k_off + h * D + d]);
    ss = fmaf(k, k, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss + 1e-6f);
  const float c = 0.60653065971263342f;      // e^(-1/2)
  float* out = packed + ((size_t)n * heads + h) * 5 * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const int e = h * D + d;
    const float k = to_f32(row[k_off + e]);
    const float za = to_f32(row[a_off + e]) + to_f32(a_bias[e]);
    const float zd = to_f32(zw[(size_t)n * zw_stride + e]) + to_f32(w_bias[e]);
    const float a = 1.f / (1.f + expf(-za));
    const float u = k * inv;
    out[d] = to_f32(row[r_off + e]);
    out[D + d] = k;
    out[2 * D + d] = expf(-c / (1.f + expf(-zd)));
    out[3 * D + d] = u;
    out[4 * D + d] = a * u;
  }
}

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// The gates of the matrix memory in two kernels.  (1) One warp per (entry, head) scans the running maximum: the two
// log gates of 32 tokens are formed side by side, one per lane, then the chain m' = max(f + m, i), which is all that
// is serial, runs over the lanes in order (an add and a max a token).  gates: [n, heads, 4] = (keep, take, m', -);
// the fourth place receives n . q from the scan.  state_m: [slots][heads], rows `slot_stride` floats apart.
template <typename T, typename W>
__global__ void __launch_bounds__(32) gate_scan_kernel(const T* __restrict__ proj, long long stride, int i_off, int f_off,
                                                       const W* __restrict__ i_bias, const W* __restrict__ f_bias,
                                                       float cap, float* __restrict__ gates, float* __restrict__ state_m,
                                                       long long slot_stride, const int* __restrict__ cu_seqlens,
                                                       const int* __restrict__ slots, int n_slots, int heads,
                                                       int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int entry = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
  const int t0 = cu_seqlens[entry], t1 = cu_seqlens[entry + 1];
  const int slot = slots[entry];
  if (slot < 0 || slot >= n_slots) {
    if (lane == 0) atomicOr(status, JV_STATUS_BAD_ROW);
    return;
  }
  float* sm = state_m + (size_t)slot * slot_stride + h;
  float m = *sm;
  const float ib = to_f32(i_bias[h]), fb = to_f32(f_bias[h]);
  auto fetch = [&](int t, float& zi, float& zf) {
    if (t < t1) {
      const T* row = proj + (size_t)t * stride;
      zi = to_f32(row[i_off + h]);
      zf = to_f32(row[f_off + h]);
    }
  };
  float zi_n = 0.f, zf_n = 0.f;
  fetch(t0 + lane, zi_n, zf_n);
  for (int base = t0; base < t1; base += 32) {
    const int t = base + lane;
    const float zi = zi_n, zf = zf_n;
    fetch(t + 32, zi_n, zf_n);                          // the next group's loads fly while this one is computed
    // a lane without a token leaves the maximum as it is: f = 0, i = -inf
    const float gi = t < t1 ? cap * tanhf((zi + ib) / cap) : -INFINITY;
    const float gf = t < t1 ? log_sigmoid(cap * tanhf((zf + fb) / cap)) : 0.f;
    float before = 0.f, after = 0.f;
#pragma unroll
    for (int l = 0; l < 32; ++l) {
      const float f = __shfl_sync(0xffffffffu, gf, l), i = __shfl_sync(0xffffffffu, gi, l);
      const float m_new = fmaxf(f + m, i);
      if (lane == l) { before = m; after = m_new; }
      m = m_new;
    }
    if (t < t1) {
      float* out = gates + ((size_t)t * heads + h) * 4;
      out[0] = expf(gf + before - after);
      out[1] = expf(gi - after);
      out[2] = after;
    }
  }
  if (lane == 0) *sm = m;
}

// (2) Per token and head, all at once: packed [n, heads, 3, D] = (q * q_scale, take * k, keep in every channel).
template <typename T>
__global__ void __launch_bounds__(128) memory_prepare_kernel(const T* __restrict__ proj, long long stride, int q_off,
                                                             int k_off, float q_scale, const float* __restrict__ gates,
                                                             float* __restrict__ packed, int heads, int D) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x, h = blockIdx.y;
  const T* row = proj + (size_t)n * stride;
  const float keep = gates[((size_t)n * heads + h) * 4], take = gates[((size_t)n * heads + h) * 4 + 1];
  float* out = packed + ((size_t)n * heads + h) * 3 * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    out[d] = to_f32(row[q_off + h * D + d]) * q_scale;
    out[D + d] = take * to_f32(row[k_off + h * D + d]);
    out[2 * D + d] = keep;
  }
}

// ------------------------------------------------------------------------------------------------------- scan
struct ScanParams {
  const float* packed;          // [n, heads, NV, D]
  const void* v; long long v_stride; int v_off;      // values: column v_off + head * V + col of a row of the projection
  float* out;                   // [n, heads * V]
  float* state; long long slot_stride;               // S of (slot, head) at state + slot * slot_stride + head * D * V
  const int* cu_seqlens; const int* slots;
  int n_slots, heads, D, V;
  // one more column, number V, with the value 1 for every token (the normaliser of a matrix memory): its state is
  // state_n [slots][heads * D] (rows `slot_stride` apart) and its output goes to nq[(token * heads + head) * nq_stride]
  float* state_n; float* nq; int nq_stride;
  // Long entries in segments (mode 0: every entry whole, one block column an entry).  An entry of len tokens has
  // max(1, ceil(len / seg_len)) segments; the segments of all entries are numbered in the entries' order and
  // blockIdx.x is a segment's number.  The columns of a segment's buffer, [D][v_tot] floats at (segment * heads +
  // head) * D * v_tot: the V value columns, the normaliser's (if any), then what the segment does to a state that
  // comes in: with the removal term D columns that start as the identity and take no value (the product of the
  // tokens' transitions), without it one column that starts as ones (the product of the decays, channel by channel).
  //   mode 1  every segment but an entry's last runs from a zero state and writes its buffer in seg_local; no output
  //   (then scan_combine_kernel chains them: seg_start[s + 1] = transition(s) seg_start[s] + local(s))
  //   mode 2  every segment runs from seg_start (an entry's first: from the state) and writes the outputs; an entry's
  //           last segment writes the state
  int mode, seg_len, n_entries, v_tot;
  float* seg_local; float* seg_start;
  int* status;
};

// Which entry and which of its segments the segment number g is; false if there is no such segment.
__device__ __forceinline__ bool find_segment(const int* __restrict__ cu_seqlens, int n_entries, int seg_len, int g,
                                             int& entry, int& seg, int& n_seg) {
  int acc = 0;
  for (int e = 0; e < n_entries; ++e) {
    const int len = cu_seqlens[e + 1] - cu_seqlens[e];
    const int ns = max(1, (len + seg_len - 1) / seg_len);
    if (g < acc + ns) { entry = e; seg = g - acc; n_seg = ns; return true; }
    acc += ns;
  }
  return false;
}

constexpr int SCAN_THREADS = 128;    // 4 warps of 8 columns x 4 key lanes
constexpr int SCAN_COLS = 32;

template <int KPT> struct ScanShape {
  static constexpr int ROW = 4 * (KPT + 4);          // floats of one vector in shared memory: a lane's KPT channels, 4 of padding
  static constexpr int CHUNK = KPT >= 64 ? 4 : 8;    // tokens per stage
};

__device__ __forceinline__ void cp_async_4(float* dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_16(float* dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <int KPT, bool REMOVAL, typename T>
__global__ void __launch_bounds__(SCAN_THREADS) state_scan_kernel(const ScanParams p) {
  constexpr int NV = REMOVAL ? 5 : 3;
  constexpr int ROW = ScanShape<KPT>::ROW, CHUNK = ScanShape<KPT>::CHUNK;
  extern __shared__ __align__(16) float smem[];       // [2][CHUNK][NV][ROW]
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kl = lane >> 3;                            // which quarter of the key channels
  const int col = blockIdx.z * SCAN_COLS + warp * 8 + (lane & 7);
  const int D = p.D, V = p.V;
  int entry = blockIdx.x, seg = 0, n_seg = 1;
  if (p.mode != 0 && !find_segment(p.cu_seqlens, p.n_entries, p.seg_len, blockIdx.x, entry, seg, n_seg)) return;
  if (p.mode == 1 && seg == n_seg - 1) return;         // nothing follows an entry's last segment
  int t0 = p.cu_seqlens[entry], t1 = p.cu_seqlens[entry + 1];
  if (p.mode != 0) {
    t0 += seg * p.seg_len;
    t1 = min(t1, t0 + p.seg_len);
  }
  const int slot = p.slots[entry];
  if (slot < 0 || slot >= p.n_slots) {
    if (tid == 0) atomicOr(p.status, JV_STATUS_BAD_ROW);
    return;
  }
  if (t0 >= t1) return;
  const bool is_n = !REMOVAL && p.state_n != nullptr && col == V;
  const int v_n = V + ((!REMOVAL && p.state_n != nullptr) ? 1 : 0);   // columns that belong to the state
  const int tcol = col - v_n;                          // mode 1: which column of the transition this thread carries
  const bool is_t = p.mode == 1 && tcol >= 0 && col < p.v_tot;
  const bool live = col < V || is_n || is_t;
  // element kk of this thread's column: S_g[kk * S_step] in the state, B_g[kk * v_tot] in a segment's buffer
  float* S_g = is_n ? p.state_n + (size_t)slot * p.slot_stride + (size_t)h * D
                    : p.state + (size_t)slot * p.slot_stride + (size_t)h * D * V + col;
  const size_t S_step = is_n ? 1 : V;
  const size_t B_off = ((size_t)blockIdx.x * p.heads + h) * D * p.v_tot + col;
  const bool from_state = p.mode == 0 || (p.mode == 2 && seg == 0);
  const bool to_state = p.mode == 0 || (p.mode == 2 && seg == n_seg - 1);
  float S[KPT];
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int kk = kl * KPT + i;
    float s0 = 0.f;
    if (live && kk < D) {
      if (p.mode == 1) s0 = is_t ? ((REMOVAL ? kk == tcol : true) ? 1.f : 0.f) : 0.f;
      else s0 = from_state ? S_g[(size_t)kk * S_step] : p.seg_start[B_off + (size_t)kk * p.v_tot];
    }
    S[i] = s0;
  }
  for (int i = tid; i < 2 * CHUNK * NV * ROW; i += SCAN_THREADS) smem[i] = 0.f;     // the padding stays zero
  __syncthreads();

  const T* vsrc = (const T*)p.v + p.v_off + (size_t)h * V + (col < V ? col : 0);
  auto stage = [&](int buf, int first) {
    // vectors of tokens first .. first + CHUNK - 1 (those that exist) into buffer `buf`
    const int tokens = min(CHUNK, t1 - first);
    const int per_token = NV * D;
    // a lane's KPT channels are a run in both places: 16 bytes a copy where the key size allows (rows of the packed
    // tensor then start on 16-byte boundaries), 4 bytes otherwise
    if ((D & 3) == 0) {
      // QP = 4 * KPT / 4 threads take a vector's 16-byte pieces, SCAN_THREADS / QP vectors at a time
      constexpr int QP = KPT, ROWS = SCAN_THREADS / QP;
      const int kk = (tid % QP) * 4, sub = tid / QP;
      if (kk < D) {
        float* dst = smem + (size_t)buf * CHUNK * NV * ROW + (kk / KPT) * (KPT + 4) + kk % KPT;
        const float* src = p.packed + ((size_t)first * p.heads + h) * per_token + kk;
        for (int tv = sub; tv < tokens * NV; tv += ROWS)
          cp_async_16(dst + tv * ROW, src + (size_t)(tv / NV) * p.heads * per_token + (tv % NV) * D);
      }
    } else {
      for (int tv = 0; tv < tokens * NV; ++tv) {
        float* row = smem + (size_t)(buf * CHUNK * NV + tv) * ROW;
        const float* src = p.packed + ((size_t)(first + tv / NV) * p.heads + h) * per_token + (tv % NV) * D;
        for (int kk = tid; kk < D; kk += SCAN_THREADS)
          cp_async_4(row + (kk / KPT) * (KPT + 4) + kk % KPT, src + kk);
      }
    }
    cp_async_commit();
  };
  float vr[CHUNK], vn[CHUNK];
  auto fetch_v = [&](float* dst, int first) {
#pragma unroll
    for (int t = 0; t < CHUNK; ++t)
      dst[t] = is_n ? 1.f : (col < V && first + t < t1) ? to_f32(vsrc[(size_t)(first + t) * p.v_stride]) : 0.f;
  };
  stage(0, t0);
  fetch_v(vr, t0);
  int buf = 0;
  for (int first = t0; first < t1; first += CHUNK, buf ^= 1) {
    cp_async_wait_all();
    __syncthreads();                                   // this chunk has landed; the other buffer is free
    if (first + CHUNK < t1) {
      stage(buf ^ 1, first + CHUNK);
      fetch_v(vn, first + CHUNK);
    }
    const int tokens = min(CHUNK, t1 - first);
    // one token: everything it needs is in shared memory and registers
    auto token = [&](const int t, const float v) {
      const float* vec = smem + (size_t)(buf * CHUNK + t) * NV * ROW + kl * (KPT + 4);
      float dot = 0.f;
      if (REMOVAL) {
#pragma unroll
        for (int i = 0; i < KPT; i += 4) {
          const float4 u = *reinterpret_cast<const float4*>(vec + 3 * ROW + i);
          dot = fmaf(u.x, S[i], dot); dot = fmaf(u.y, S[i + 1], dot);
          dot = fmaf(u.z, S[i + 2], dot); dot = fmaf(u.w, S[i + 3], dot);
        }
        dot += __shfl_xor_sync(0xffffffffu, dot, 8);
        dot += __shfl_xor_sync(0xffffffffu, dot, 16);
      }
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < KPT; i += 4) {
        const float4 r = *reinterpret_cast<const float4*>(vec + i);
        const float4 k = *reinterpret_cast<const float4*>(vec + ROW + i);
        const float4 w = *reinterpret_cast<const float4*>(vec + 2 * ROW + i);
        float s0 = fmaf(k.x, v, w.x * S[i]), s1 = fmaf(k.y, v, w.y * S[i + 1]);
        float s2 = fmaf(k.z, v, w.z * S[i + 2]), s3 = fmaf(k.w, v, w.w * S[i + 3]);
        if (REMOVAL) {
          const float4 b = *reinterpret_cast<const float4*>(vec + 4 * ROW + i);
          s0 = fmaf(-b.x, dot, s0); s1 = fmaf(-b.y, dot, s1); s2 = fmaf(-b.z, dot, s2); s3 = fmaf(-b.w, dot, s3);
        }
        S[i] = s0; S[i + 1] = s1; S[i + 2] = s2; S[i + 3] = s3;
        o = fmaf(r.x, s0, o); o = fmaf(r.y, s1, o); o = fmaf(r.z, s2, o); o = fmaf(r.w, s3, o);
      }
      o += __shfl_xor_sync(0xffffffffu, o, 8);
      o += __shfl_xor_sync(0xffffffffu, o, 16);
      if (kl == 0 && live && p.mode != 1) {
        if (is_n) p.nq[((size_t)(first + t) * p.heads + h) * p.nq_stride] = o;
        else p.out[(size_t)(first + t) * p.heads * V + (size_t)h * V + col] = o;
      }
    };
    if (REMOVAL && tokens == CHUNK) {
      // with the removal term a token is a long chain of dependent steps (dot, two shuffles, update, dot, two shuffles):
      // a whole stage is unrolled, so that the reduction and the store of a token's output run under the next token's
      // first dot product (measured: 1,024 -> 936 us for 2,048 tokens of 32 heads of 64).  Without the term the unrolled
      // form needs 254 registers where the loop needs 168, and two blocks a multiprocessor are slower than three.
#pragma unroll
      for (int t = 0; t < CHUNK; ++t) token(t, vr[t]);
    } else {
      for (int t = 0; t < tokens; ++t) token(t, vr[t]);
    }
#pragma unroll
    for (int t = 0; t < CHUNK; ++t) vr[t] = vn[t];
  }
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int kk = kl * KPT + i;
    if (live && kk < D) {
      if (p.mode == 1) p.seg_local[B_off + (size_t)kk * p.v_tot] = S[i];
      else if (to_state) S_g[(size_t)kk * S_step] = S[i];
    }
  }
}

// Chains the segments of an entry: from the state that the entry brings, seg_start[s + 1] = T_s seg_start[s] + local_s,
// where T_s is what segment s does to a state that comes in (seg_local's last columns).
// Without the removal term T_s is diagonal (one column of decay products): every element of the state is a chain of
// its own, one thread an element, grid (entry, head, blocks over D * columns).
__global__ void __launch_bounds__(128) scan_combine_diag_kernel(const ScanParams p) {
  pdl_trigger();
  pdl_wait();
  const int entry = blockIdx.x, h = blockIdx.y;
  const int D = p.D, V = p.V;
  const int v_n = V + (p.state_n != nullptr ? 1 : 0);
  const int idx = blockIdx.z * 128 + threadIdx.x;
  if (idx >= D * v_n) return;
  const int kk = idx / v_n, col = idx - kk * v_n;
  const int len = p.cu_seqlens[entry + 1] - p.cu_seqlens[entry];
  const int n_seg = max(1, (len + p.seg_len - 1) / p.seg_len);
  if (n_seg < 2) return;
  const int slot = p.slots[entry];
  if (slot < 0 || slot >= p.n_slots) return;             // the scan reports it
  int g0 = 0;                                            // the number of the entry's first segment
  for (int e = 0; e < entry; ++e) g0 += max(1, (p.cu_seqlens[e + 1] - p.cu_seqlens[e] + p.seg_len - 1) / p.seg_len);
  float S = (col == V) ? p.state_n[(size_t)slot * p.slot_stride + (size_t)h * D + kk]
                       : p.state[(size_t)slot * p.slot_stride + (size_t)h * D * V + (size_t)kk * V + col];
  const size_t seg_floats = (size_t)p.heads * D * p.v_tot;
  const float* local = p.seg_local + ((size_t)g0 * p.heads + h) * D * p.v_tot + (size_t)kk * p.v_tot;
  float* start = p.seg_start + ((size_t)(g0 + 1) * p.heads + h) * D * p.v_tot + (size_t)kk * p.v_tot + col;
  float t_next = local[v_n], l_next = local[col];
  for (int sg = 0; sg + 1 < n_seg; ++sg) {
    const float t = t_next, l = l_next;
    if (sg + 2 < n_seg) {                                // the next segment's numbers are under way
      t_next = local[(size_t)(sg + 1) * seg_floats + v_n];
      l_next = local[(size_t)(sg + 1) * seg_floats + col];
    }
    S = fmaf(t, S, l);
    start[(size_t)sg * seg_floats] = S;
  }
}

// With the removal term T_s is a [D][D] matrix.  One block per (entry, head, 32 columns); a thread keeps the rows
// tid / 32, tid / 32 + 4, ... of its column.  Per segment the matrix comes into shared memory once (all threads, 16
// bytes a load) beside the block's columns, and a row's product reads four of its numbers at a time.
constexpr int COMBINE_ROWS = 64;     // rows a thread: keys up to 256
__global__ void __launch_bounds__(128) scan_combine_kernel(const ScanParams p) {
  extern __shared__ __align__(16) float csm[];           // cols [D][32], local [D][32], T [D][DP], DP = D rounded up to 4, plus 4
  pdl_trigger();
  pdl_wait();
  const int entry = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int lane = tid & 31, col = blockIdx.z * 32 + lane, r0 = tid >> 5;
  const int D = p.D, V = p.V;
  const int DP = ((D + 3) & ~3) + 4;
  float* cols = csm;
  float* Ls = csm + (size_t)D * 32;
  float* Ts = csm + (size_t)D * 64;
  const int len = p.cu_seqlens[entry + 1] - p.cu_seqlens[entry];
  const int n_seg = max(1, (len + p.seg_len - 1) / p.seg_len);
  if (n_seg < 2) return;
  const int slot = p.slots[entry];
  if (slot < 0 || slot >= p.n_slots) return;             // the scan reports it
  int g0 = 0;
  for (int e = 0; e < entry; ++e) g0 += max(1, (p.cu_seqlens[e + 1] - p.cu_seqlens[e] + p.seg_len - 1) / p.seg_len);
  const bool live = col < V;
  const float* S_g = p.state + (size_t)slot * p.slot_stride + (size_t)h * D * V + col;
  float S[COMBINE_ROWS];
#pragma unroll
  for (int i = 0; i < COMBINE_ROWS; ++i) {
    const int kk = r0 + 4 * i;
    S[i] = (live && kk < D) ? S_g[(size_t)kk * V] : 0.f;
  }
  for (int i = tid; i < D * DP; i += 128) Ts[i] = 0.f;   // the padding stays zero
  for (int sg = 0; sg + 1 < n_seg; ++sg) {
    const size_t base = ((size_t)(g0 + sg) * p.heads + h) * D * p.v_tot;
    const float* local = p.seg_local + base;
    __syncthreads();                                     // the segment before has read the columns and the matrix
#pragma unroll
    for (int i = 0; i < COMBINE_ROWS; ++i) {
      const int kk = r0 + 4 * i;
      if (kk < D) cols[kk * 32 + lane] = S[i];
    }
    // the segment's matrix and the block's columns of its local result come in as asynchronous copies: no load waits
    // for another
    for (int i = tid; i < D * D; i += 128) {
      const int kk = i / D, j = i - kk * D;
      cp_async_4(Ts + kk * DP + j, local + (size_t)kk * p.v_tot + V + j);
    }
    if (live)
      for (int kk = r0; kk < D; kk += 4) cp_async_4(Ls + kk * 32 + lane, local + (size_t)kk * p.v_tot + col);
    cp_async_commit();
    cp_async_wait_all();
    __syncthreads();
#pragma unroll
    for (int i = 0; i < COMBINE_ROWS; ++i) {
      const int kk = r0 + 4 * i;
      if (kk < D) {
        const float* trow = Ts + kk * DP;
        float a0 = live ? Ls[kk * 32 + lane] : 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        for (int j = 0; j < D; j += 4) {                 // past D the matrix's padding is zero and the columns are finite
          const float4 t4 = *reinterpret_cast<const float4*>(trow + j);
          a0 = fmaf(t4.x, cols[j * 32 + lane], a0);
          if (j + 1 < D) a1 = fmaf(t4.y, cols[(j + 1) * 32 + lane], a1);
          if (j + 2 < D) a2 = fmaf(t4.z, cols[(j + 2) * 32 + lane], a2);
          if (j + 3 < D) a3 = fmaf(t4.w, cols[(j + 3) * 32 + lane], a3);
        }
        S[i] = (a0 + a1) + (a2 + a3);
      }
    }
    float* start = p.seg_start + base + (size_t)D * p.v_tot * p.heads;      // the buffer of segment g0 + sg + 1
#pragma unroll
    for (int i = 0; i < COMBINE_ROWS; ++i) {
      const int kk = r0 + 4 * i;
      if (live && kk < D) start[(size_t)kk * p.v_tot + col] = S[i];
    }
  }
}

template <int KPT, bool REMOVAL, typename T>
int launch_scan(const ScanParams& p, int entries, cudaStream_t stream) {
  constexpr int NV = REMOVAL ? 5 : 3;
  const size_t smem = sizeof(float) * 2 * ScanShape<KPT>::CHUNK * NV * ScanShape<KPT>::ROW;
  auto kern = state_scan_kernel<KPT, REMOVAL, T>;
  static bool done[JV_MAX_DEVICES] = {};
  if (!jv_once_per_device(done, [&] {
        return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
      }))
    return JV_ERR_UNSUPPORTED;
  const int cols = p.V + ((!REMOVAL && p.state_n != nullptr) ? 1 : 0);
  if (p.mode == 0)
    return jv_launch(kern, dim3(entries, p.heads, (cols + SCAN_COLS - 1) / SCAN_COLS), dim3(SCAN_THREADS), smem, stream, p);
  // in segments: `entries` is then the largest number of segments there can be
  ScanParams q = p;
  q.mode = 1;
  int rc = jv_launch(kern, dim3(entries, p.heads, (p.v_tot + SCAN_COLS - 1) / SCAN_COLS), dim3(SCAN_THREADS), smem, stream, q);
  if (rc != JV_OK) return rc;
  if (REMOVAL) {
    const size_t csmem = sizeof(float) * ((size_t)p.D * 64 + (size_t)p.D * (((p.D + 3) & ~3) + 4));
    if (csmem > 200 * 1024) return JV_ERR_UNSUPPORTED;
    static bool cdone[JV_MAX_DEVICES] = {};
    if (!jv_once_per_device(cdone, [&] {
          return cudaFuncSetAttribute(scan_combine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess;
        }))
      return JV_ERR_UNSUPPORTED;
    rc = jv_launch(scan_combine_kernel, dim3(p.n_entries, p.heads, (cols + 31) / 32), dim3(128), csmem, stream, q);
  } else {
    rc = jv_launch(scan_combine_diag_kernel, dim3(p.n_entries, p.heads, (p.D * cols + 127) / 128), dim3(128), 0, stream, q);
  }
  if (rc != JV_OK) return rc;
  q.mode = 2;
  return jv_launch(kern, dim3(entries, p.heads, (cols + SCAN_COLS - 1) / SCAN_COLS), dim3(SCAN_THREADS), smem, stream, q);
}

template <bool REMOVAL, typename T>
int dispatch_scan(const ScanParams& p, int entries, cudaStream_t stream) {
  const int kpt = (p.D + 3) / 4;
  if (kpt <= 4) return launch_scan<4, REMOVAL, T>(p, entries, stream);
  if (kpt <= 8) return launch_scan<8, REMOVAL, T>(p, entries, stream);
  if (kpt <= 16) return launch_scan<16, REMOVAL, T>(p, entries, stream);
  if (kpt <= 32) return launch_scan<32, REMOVAL, T>(p, entries, stream);
  if (kpt <= 64) return launch_scan<64, REMOVAL, T>(p, entries, stream);
  return JV_ERR_UNSUPPORTED;
}

// ----------------------------------------------------------------------------------------------------- finish
template <typename T, typename W>
__global__ void __launch_bounds__(128) head_norm_gate_kernel(const float* __restrict__ o, const W* __restrict__ weight,
                                                             const T* __restrict__ gate, long long gate_stride,
                                                             T* __restrict__ out, long long out_stride, int heads, int V,
                                                             float eps, const float* __restrict__ gates) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x, h = blockIdx.y;
  const float* src = o + ((size_t)n * heads + h) * V;
  // a matrix memory's output is first divided by max(|n . q|, exp(-m)) + 1e-6 (gates: [n, heads, 4] = (-, -, m, n . q))
  float den = 1.f;
  if (gates != nullptr) {
    const float* g = gates + ((size_t)n * heads + h) * 4;
    den = 1.f / (fmaxf(fabsf(g[3]), expf(-g[2])) + 1e-6f);
  }
  float ss = 0.f;
  for (int j = threadIdx.x; j < V; j += blockDim.x) ss = fmaf(src[j] * den, src[j] * den, ss);
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)V + eps);
  for (int j = threadIdx.x; j < V; j += blockDim.x) {
    float y = src[j] * den * inv * to_f32(weight[h * V + j]);
    if (gate != nullptr) y *= 1.f / (1.f + expf(-to_f32(gate[(size_t)n * gate_stride + h * V + j])));
    out[(size_t)n * out_stride + h * V + j] = from_f32<T>(y);
  }
}

}  // namespace

// proj: [n] rows of `stride` elements of dtype `dtype` holding r, k and the removal gate's pre-activation at the given
// columns (heads * D each); zw: [n] rows of the decay's pre-activation; a_bias, w_bias: [heads * D] of dtype `w_dtype`;
// packed: [n, heads, 5, D] float.
JV_EXPORT int jv_delta_prepare(const void* proj, int dtype, long long stride, int r_off, int k_off, int a_off,
                               const void* zw, long long zw_stride, const void* a_bias, const void* w_bias, int w_dtype,
                               float* packed, int n, int heads, int D, cudaStream_t stream) {
  if (n == 0) return JV_OK;
  JV_DISPATCH_DTYPE(dtype, T, JV_DISPATCH_DTYPE(w_dtype, W, return jv_launch(
      delta_prepare_kernel<T, W>, dim3(n, heads), dim3(D > 64 ? 128 : 64), 0, stream, (const T*)proj, stride, r_off, k_off,
      a_off, (const T*)zw, zw_stride, (const W*)a_bias, (const W*)w_bias, packed, heads, D)));
  return JV_ERR_UNSUPPORTED;
}

// proj as above with q, k (heads * D each) and the two gates' pre-activations (heads each) at the given columns;
// gates: [n, heads, 4] float (keep, take, running maximum; the fourth place is left for the scan's n . q); packed:
// [n, heads, 3, D] float; state_m: the running maximum of slot 0, rows `slot_stride` floats apart.
JV_EXPORT int jv_memory_gates(const void* proj, int dtype, long long stride, int q_off, int k_off, int i_off, int f_off,
                              const void* i_bias, const void* f_bias, int w_dtype, float cap, float q_scale, float* gates,
                              float* packed, float* state_m, long long slot_stride, const int* cu_seqlens,
                              const int* slots, int n_slots, int entries, int n, int heads, int D, int* status,
                              cudaStream_t stream) {
  if (entries == 0 || n == 0) return JV_OK;
  JV_DISPATCH_DTYPE(dtype, T, JV_DISPATCH_DTYPE(w_dtype, W, {
    const int rc = jv_launch(gate_scan_kernel<T, W>, dim3(entries, heads), dim3(32), 0, stream, (const T*)proj, stride,
                             i_off, f_off, (const W*)i_bias, (const W*)f_bias, cap, gates, state_m, slot_stride,
                             cu_seqlens, slots, n_slots, heads, status);
    if (rc != JV_OK) return rc;
    return jv_launch(memory_prepare_kernel<T>, dim3(n, heads), dim3(D > 64 ? 128 : 64), 0, stream, (const T*)proj, stride,
                     q_off, k_off, q_scale, (const float*)gates, packed, heads, D);
  }));
  return JV_ERR_UNSUPPORTED;
}

// The scan itself; `removal`: the packed rows hold (r, k, w, u, b), else (r, k, w).  v: rows of the projection.
// state_n (or null; without removal only): [slots][heads * D], rows `slot_stride` apart, the state of one more column
// whose value is 1 at every token; its outputs go to nq[(token * heads + head) * nq_stride].
// seg_len > 0: entries longer than seg_len tokens run in segments of that many, side by side (see ScanParams): three
// launches; seg_local and seg_start hold max_segments * heads * D * (V + (state_n ? 1 : 0) + (removal ? D : 1)) floats
// each, and max_segments is at least the number of segments of all entries together.
JV_EXPORT int jv_state_scan(const float* packed, int removal, const void* v, int dtype, long long v_stride, int v_off,
                            float* out, float* state, long long slot_stride, const int* cu_seqlens, const int* slots,
                            int n_slots, int entries, int heads, int D, int V, float* state_n, float* nq, int nq_stride,
                            int seg_len, int max_segments, float* seg_local, float* seg_start, int* status,
                            cudaStream_t stream) {
  if (entries == 0) return JV_OK;
  if (state_n != nullptr && (removal || nq == nullptr)) return JV_ERR_UNSUPPORTED;
  if (seg_len > 0 && (seg_local == nullptr || seg_start == nullptr || max_segments < entries || D > 4 * COMBINE_ROWS))
    return JV_ERR_UNSUPPORTED;
  ScanParams p;
  p.mode = seg_len > 0 ? 1 : 0; p.seg_len = seg_len; p.n_entries = entries; p.seg_local = seg_local; p.seg_start = seg_start;
  p.v_tot = V + (state_n != nullptr ? 1 : 0) + (removal ? D : 1);
  if (seg_len > 0) entries = max_segments;
  p.state_n = state_n; p.nq = nq; p.nq_stride = nq_stride;
  p.packed = packed; p.v = v; p.v_stride = v_stride; p.v_off = v_off; p.out = out; p.state = state;
  p.slot_stride = slot_stride; p.cu_seqlens = cu_seqlens; p.slots = slots; p.n_slots = n_slots; p.heads = heads;
  p.D = D; p.V = V; p.status = status;
  JV_DISPATCH_DTYPE(dtype, T, {
    return removal ? dispatch_scan<true, T>(p, entries, stream) : dispatch_scan<false, T>(p, entries, stream);
  });
  return JV_ERR_UNSUPPORTED;
}

// o: [n, heads * V] float; weight: [heads * V] of dtype `w_dtype`; gate: rows of `gate_stride` elements (or null);
// out: rows of `out_stride` elements, both of dtype `dtype`.
JV_EXPORT int jv_head_norm_gate(const float* o, const void* weight, int w_dtype, const void* gate, long long gate_stride,
                                void* out, int dtype, long long out_stride, int n, int heads, int V, float eps,
                                const float* gates, cudaStream_t stream) {
  if (n == 0) return JV_OK;
  JV_DISPATCH_DTYPE(dtype, T, JV_DISPATCH_DTYPE(w_dtype, W, return jv_launch(
      head_norm_gate_kernel<T, W>, dim3(n, heads), dim3(V > 64 ? 128 : 64), 0, stream, o, (const W*)weight, (const T*)gate,
      gate_stride, (T*)out, out_stride, heads, V, eps, gates)));
  return JV_ERR_UNSUPPORTED;
}
