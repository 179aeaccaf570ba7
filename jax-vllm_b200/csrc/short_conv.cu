// A short causal convolution over time on each channel, with the last taps - 1 inputs of every sequence kept as
// state, so that a sequence may be cut into steps anywhere:
//
//   conv_t[c] = sum_j w[c, j] * in_(t - taps + 1 + j)[c]        (the last column weighs the current token; inputs
//                                                                before the sequence's start are zero)
//   out_t[c]  = act(conv_t[c] + bias[c])            act: none or silu
//           or  in_t[c] + conv_t[c]                 `residual`: the convolution is added to what it reads
//
// state[slot, j, c], j < taps - 1, holds the input at the sequence's position (tokens so far) - (taps - 1) + j; a
// fresh slot is zero, which is the zero padding.  All arithmetic is 32-bit, whatever the types of in and out.
//
// A thread owns one channel of one segment of SEG tokens of one entry and slides a window of taps - 1 registers over
// it (SEG is at least taps - 1).  Segments are counted per entry, so only an entry's first segment reads the state; the thread of that segment
// is also the ONE writer of the entry's state for its channel: it has the old state in its window before it writes
// the new one (the entry's last taps - 1 inputs, or old state shifted where the entry is shorter), so no other
// thread reads what it overwrites.  Blocks find their (entry, segment) from cu_seqlens; the grid is an upper bound,
// n / SEG + entries, and blocks beyond the last segment leave.
#include "common.cuh"

namespace {
constexpr int SEG = 32;
constexpr int THREADS = 128;
constexpr int BATCH = 8;       // inputs a thread asks for before it uses the first

struct ConvParams {
  const void* in; long long in_stride;
  void* out; long long out_stride;
  const void* w; const void* bias;
  float* state; long long state_stride;      // elements between slots
  const int* cu_seqlens; const int* slots;
  int n_entries, n_slots, channels, act, residual;
  int* status;
};

template <typename TI, typename TO, typename TW, int TAPS>
__global__ void __launch_bounds__(THREADS) short_conv_kernel(const ConvParams p) {
  pdl_trigger();
  pdl_wait();
  // which segment of which entry
  int entry = -1, seg = 0, before = 0;
  for (int e = 0; e < p.n_entries; ++e) {
    const int q = p.cu_seqlens[e + 1] - p.cu_seqlens[e];
    const int segs = (q + SEG - 1) / SEG;
    if ((int)blockIdx.x < before + segs) { entry = e; seg = blockIdx.x - before; break; }
    before += segs;
  }
  if (entry < 0) return;
  const int c = blockIdx.y * THREADS + threadIdx.x;
  if (c >= p.channels) return;
  const int t_begin = p.cu_seqlens[entry], q = p.cu_seqlens[entry + 1] - t_begin;
  const int i0 = seg * SEG, i1 = min(q, i0 + SEG);
  constexpr int K = TAPS - 1;
  const int slot = K > 0 ? p.slots[entry] : 0;        // one tap keeps nothing
  if (K > 0 && (slot < 0 || slot >= p.n_slots)) {
    if (threadIdx.x == 0) atomicOr(p.status, JV_STATUS_BAD_ROW);
    return;
  }
  const TI* in = (const TI*)p.in + c;
  TO* out = (TO*)p.out + c;
  float* st = K > 0 ? p.state + (size_t)slot * p.state_stride + c : nullptr;
  float wt[TAPS];
#pragma unroll
  for (int j = 0; j < TAPS; ++j) wt[j] = to_f32(((const TW*)p.w)[(size_t)c * TAPS + j]);
  const float b = p.bias != nullptr ? to_f32(((const TW*)p.bias)[c]) : 0.f;
  float win[K > 0 ? K : 1];          // win[k]: the input at offset i0 - K + k of the entry
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int i = i0 - K + k;
    win[k] = i >= 0 ? to_f32(in[(size_t)(t_begin + i) * p.in_stride]) : st[(size_t)(K + i) * p.channels];
  }
  if (seg == 0) {
    // the state after this step: the last K inputs of (old state, this entry's tokens)
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int i = q - K + j;
      float v;
      if (i >= 0) {
        v = to_f32(in[(size_t)(t_begin + i) * p.in_stride]);
      } else {
        v = 0.f;
#pragma unroll
        for (int k = 0; k < K; ++k) if (k == K + i) v = win[k];      // old state j + q
      }
      st[(size_t)j * p.channels] = v;
    }
  }
  // BATCH tokens at a time: their loads are under way together (a thread's tokens lie a whole row apart)
  for (int i = i0; i < i1; i += BATCH) {
    float xs[BATCH];
#pragma unroll
    for (int u = 0; u < BATCH; ++u) xs[u] = i + u < i1 ? to_f32(in[(size_t)(t_begin + i + u) * p.in_stride]) : 0.f;
#pragma unroll
    for (int u = 0; u < BATCH; ++u) {
      if (i + u >= i1) break;
      const float x = xs[u];
      float acc = wt[K] * x;
#pragma unroll
      for (int k = 0; k < K; ++k) acc = fmaf(wt[k], win[k], acc);
#pragma unroll
      for (int k = 0; k + 1 < K; ++k) win[k] = win[k + 1];
      if (K > 0) win[K - 1] = x;
      float y = p.residual ? x + acc : acc + b;
      if (p.act == 1) y = y / (1.f + expf(-y));
      out[(size_t)(t_begin + i + u) * p.out_stride] = from_f32<TO>(y);
    }
  }
}

template <typename TI, typename TO, typename TW>
int launch_taps(const ConvParams& p, int taps, dim3 grid, cudaStream_t stream) {
  switch (taps) {
    case 1: return jv_launch(short_conv_kernel<TI, TO, TW, 1>, grid, dim3(THREADS), 0, stream, p);
    case 2: return jv_launch(short_conv_kernel<TI, TO, TW, 2>, grid, dim3(THREADS), 0, stream, p);
    case 3: return jv_launch(short_conv_kernel<TI, TO, TW, 3>, grid, dim3(THREADS), 0, stream, p);
    case 4: return jv_launch(short_conv_kernel<TI, TO, TW, 4>, grid, dim3(THREADS), 0, stream, p);
    case 5: return jv_launch(short_conv_kernel<TI, TO, TW, 5>, grid, dim3(THREADS), 0, stream, p);
    case 6: return jv_launch(short_conv_kernel<TI, TO, TW, 6>, grid, dim3(THREADS), 0, stream, p);
    case 7: return jv_launch(short_conv_kernel<TI, TO, TW, 7>, grid, dim3(THREADS), 0, stream, p);
    case 8: return jv_launch(short_conv_kernel<TI, TO, TW, 8>, grid, dim3(THREADS), 0, stream, p);
    default: return JV_ERR_UNSUPPORTED;
  }
}
}  // namespace

JV_EXPORT int jv_short_conv_max_taps() { return 8; }

// in: [n, in_stride] of in_dtype (the first `channels` columns from the pointer); out: [n, out_stride] of out_dtype;
// w: [channels, taps] and bias [channels] (or null) of w_dtype; state: float [n_slots][taps - 1][channels], slots
// `state_stride` elements apart (null only with taps == 1); cu_seqlens [n_entries + 1], slots [n_entries].
// act: 0 none, 1 silu.  residual: out = in + conv (no bias, no activation on the sum unless act says so).
JV_EXPORT int jv_short_conv(const void* in, int in_dtype, long long in_stride, void* out, int out_dtype,
                            long long out_stride, const void* w, const void* bias, int w_dtype, float* state,
                            long long state_stride, const int* cu_seqlens, const int* slots, int n_entries, int n_slots,
                            int n_tokens, int channels, int taps, int act, int residual, int* status,
                            cudaStream_t stream) {
  if (n_tokens == 0 || n_entries == 0 || channels == 0) return JV_OK;
  if (taps < 1 || taps > 8 || act < 0 || act > 1 || (taps > 1 && state == nullptr)) return JV_ERR_UNSUPPORTED;
  ConvParams p;
  p.in = in; p.in_stride = in_stride; p.out = out; p.out_stride = out_stride; p.w = w; p.bias = residual ? nullptr : bias;
  p.state = state; p.state_stride = state_stride; p.cu_seqlens = cu_seqlens; p.slots = slots; p.n_entries = n_entries;
  p.n_slots = n_slots; p.channels = channels; p.act = act; p.residual = residual ? 1 : 0; p.status = status;
  const dim3 grid(n_tokens / SEG + n_entries, (channels + THREADS - 1) / THREADS);
  JV_DISPATCH_DTYPE(in_dtype, TI, JV_DISPATCH_DTYPE(out_dtype, TO, JV_DISPATCH_DTYPE(w_dtype, TW,
      return launch_taps<TI, TO, TW>(p, taps, grid, stream))));
  return JV_ERR_UNSUPPORTED;
}
