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
  int* status;
};

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
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <int KPT, bool REMOVAL, typename T>
__global__ void __launch_bounds__(SCAN_THREADS) state_scan_kernel(const ScanParams p) {
  constexpr int NV = REMOVAL ? 5 : 3;
  constexpr int ROW = ScanShape<KPT>::ROW, CHUNK = ScanShape<KPT>::CHUNK;
  extern __shared__ __align__(16) float smem[];       // [2][CHUNK][NV][ROW]
  pdl_trigger();
  pdl_wait();
  const int entry = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kl = lane >> 3;                            // which quarter of the key channels
  const int col = blockIdx.z * SCAN_COLS + warp * 8 + (lane & 7);
  const int D = p.D, V = p.V;
  const int t0 = p.cu_seqlens[entry], t1 = p.cu_seqlens[entry + 1];
  const int slot = p.slots[entry];
  if (slot < 0 || slot >= p.n_slots) {
    if (tid == 0) atomicOr(p.status, JV_STATUS_BAD_ROW);
    return;
  }
  if (t0 >= t1) return;
  const bool is_n = !REMOVAL && p.state_n != nullptr && col == V;
  const bool live = col < V || is_n;
  // element kk of this thread's column: S_g[kk * S_step]
  float* S_g = is_n ? p.state_n + (size_t)slot * p.slot_stride + (size_t)h * D
                    : p.state + (size_t)slot * p.slot_stride + (size_t)h * D * V + col;
  const size_t S_step = is_n ? 1 : V;
  float S[KPT];
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int kk = kl * KPT + i;
    S[i] = (live && kk < D) ? S_g[(size_t)kk * S_step] : 0.f;
  }
  for (int i = tid; i < 2 * CHUNK * NV * ROW; i += SCAN_THREADS) smem[i] = 0.f;     // the padding stays zero
  __syncthreads();

  const T* vsrc = (const T*)p.v + p.v_off + (size_t)h * V + (col < V ? col : 0);
  auto stage = [&](int buf, int first) {
    // vectors of tokens first .. first + CHUNK - 1 (those that exist) into buffer `buf`
    const int tokens = min(CHUNK, t1 - first);
    const int per_token = NV * D;
    for (int i = tid; i < tokens * per_token; i += SCAN_THREADS) {
      const int t = i / per_token, r = i - t * per_token;
      const int v = r / D, kk = r - v * D;
      float* dst = smem + ((size_t)(buf * CHUNK + t) * NV + v) * ROW + (kk / KPT) * (KPT + 4) + kk % KPT;
      cp_async_4(dst, p.packed + ((size_t)(first + t) * p.heads + h) * per_token + r);
    }
    cp_async_commit();
  };
  float vr[CHUNK], vn[CHUNK];
  auto fetch_v = [&](float* dst, int first) {
#pragma unroll
    for (int t = 0; t < CHUNK; ++t)
      dst[t] = is_n ? 1.f : (first + t < t1) ? to_f32(vsrc[(size_t)(first + t) * p.v_stride]) : 0.f;
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
    for (int t = 0; t < tokens; ++t) {
      const float* vec = smem + (size_t)(buf * CHUNK + t) * NV * ROW + kl * (KPT + 4);
      const float v = vr[t];
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
      if (kl == 0 && live) {
        if (is_n) p.nq[((size_t)(first + t) * p.heads + h) * p.nq_stride] = o;
        else p.out[(size_t)(first + t) * p.heads * V + (size_t)h * V + col] = o;
      }
    }
#pragma unroll
    for (int t = 0; t < CHUNK; ++t) vr[t] = vn[t];
  }
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    const int kk = kl * KPT + i;
    if (live && kk < D) S_g[(size_t)kk * S_step] = S[i];
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
  return jv_launch(kern, dim3(entries, p.heads, (cols + SCAN_COLS - 1) / SCAN_COLS), dim3(SCAN_THREADS), smem, stream, p);
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
JV_EXPORT int jv_state_scan(const float* packed, int removal, const void* v, int dtype, long long v_stride, int v_off,
                            float* out, float* state, long long slot_stride, const int* cu_seqlens, const int* slots,
                            int n_slots, int entries, int heads, int D, int V, float* state_n, float* nq, int nq_stride,
                            int* status, cudaStream_t stream) {
  if (entries == 0) return JV_OK;
  if (state_n != nullptr && (removal || nq == nullptr)) return JV_ERR_UNSUPPORTED;
  ScanParams p;
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
