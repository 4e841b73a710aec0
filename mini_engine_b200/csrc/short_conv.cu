// A short causal convolution over time on each channel, with the last inputs of every request kept as state.
//
// out_t = [h_t +] sum_j w[:, j] * h_(t - taps + 1 + j), j = 0 .. taps-1, zeros before the request's first token.
// A request's portion of a step starts at position ``start`` = context length - tokens in the step; inputs at
// positions before ``start`` come from the request's state slot, which holds the last taps-1 inputs (state row k is
// position start - (taps-1) + k).  A second kernel then stores the last taps-1 inputs of the portion (moving old
// state rows up when the portion is shorter than taps-1).  A slot is never read for positions below 0, so a slot
// that another request used before needs no clearing.  Inputs, weights and state are float32.
#include "common.cuh"

template <typename TO>
__global__ void __launch_bounds__(256)
short_conv_kernel(const float* __restrict__ h, const float* __restrict__ wt, const float* __restrict__ state,
                  const int* __restrict__ token_req, const int* __restrict__ cu_seqlens,
                  const int* __restrict__ context_lens, const int* __restrict__ state_slots, TO* __restrict__ out,
                  int W, int taps, int add_input) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int w = blockIdx.y * blockDim.x + threadIdx.x;
  if (w >= W) return;
  const int b = token_req[t];
  const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0;
  const int start = context_lens[b] - q_len;
  const int i = t - tok0;                         // local index in the portion
  const int slot = state_slots[b];
  float acc = add_input ? h[(int64_t)t * W + w] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int src = i - (taps - 1) + j;           // local index of the input
    if (start + src < 0) continue;                // before the request's first token
    float v;
    if (src >= 0) {
      v = h[(int64_t)(tok0 + src) * W + w];
    } else {
      if (slot < 0) continue;
      v = state[((int64_t)slot * (taps - 1) + (src + taps - 1)) * W + w];
    }
    acc = fmaf(wt[(int64_t)w * taps + j], v, acc);
  }
  out[(int64_t)t * W + w] = from_f<TO>(acc);
}

__global__ void __launch_bounds__(256)
short_conv_state_kernel(const float* __restrict__ h, float* __restrict__ state, const int* __restrict__ cu_seqlens,
                        const int* __restrict__ context_lens, const int* __restrict__ state_slots, int W, int taps) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const int w = blockIdx.y * blockDim.x + threadIdx.x;
  if (w >= W) return;
  const int slot = state_slots[b];
  if (slot < 0) return;
  const int tok0 = cu_seqlens[b], n = cu_seqlens[b + 1] - tok0;
  if (n <= 0) return;
  const int start = context_lens[b] - n;
  float* st = state + (int64_t)slot * (taps - 1) * W + w;
  // Row k takes the input at local index n - (taps-1) + k.  Old rows are read at k + n > k, rows are written in
  // ascending order, so a thread never reads a row it has already replaced.
  for (int k = 0; k < taps - 1; ++k) {
    const int src = n - (taps - 1) + k;
    float v = 0.f;
    if (src >= 0) v = h[(int64_t)(tok0 + src) * W + w];
    else if (start + src >= 0) v = st[(int64_t)(src + taps - 1) * W];
    st[(int64_t)k * W] = v;
  }
}

// h: [T, W] float32.  wt: [W, taps] float32.  state: [slots, taps-1, W] float32 (unused when taps == 1).
// out: [T, W] of out_dtype.  update_state != 0 also runs the second kernel.
ME_API int me_short_conv(const float* h, const float* wt, float* state, const int* token_req, const int* cu_seqlens,
                         const int* context_lens, const int* state_slots, void* out, int out_dtype, int T, int B, int W,
                         int taps, int add_input, int update_state, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && B > 0 && W > 0 && taps >= 1, "me_short_conv: bad sizes T=%d B=%d W=%d taps=%d", T, B, W, taps);
  ME_REQUIRE(taps == 1 || state != nullptr, "me_short_conv: %d taps need a state", taps);
  const int threads = W >= 256 ? 256 : 64;
  dim3 grid(T, (W + threads - 1) / threads);
  ME_DISPATCH_DTYPE(out_dtype, TO,
                    me_launch(short_conv_kernel<TO>, grid, dim3(threads), 0, stream, h, wt, (const float*)state, token_req,
                              cu_seqlens, context_lens, state_slots, (TO*)out, W, taps, add_input));
  ME_LAUNCH_CHECK("me_short_conv");
  if (update_state && taps > 1) {
    me_launch(short_conv_state_kernel, dim3(B, (W + threads - 1) / threads), dim3(threads), 0, stream, h, state, cu_seqlens,
              context_lens, state_slots, W, taps);
    ME_LAUNCH_CHECK("me_short_conv (state)");
  }
  return 0;
}
