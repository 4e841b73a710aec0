// Several residual streams ("hyper-connections") and the layer norm that reads them, in one pass over a token.
//
// A model may keep S copies x_1 .. x_S of the residual stream.  A sub-layer reads u = sum_s in[s] x_s, and its
// output y goes back into all streams at once: x'_r = sum_s mix[s, r] x_s + out[r] y.  The kernel applies the
// update that the sub-layer before left pending (if any), forms the next sub-layer's input u from the new
// streams and normalises it: (u - mean) / sqrt(var + eps) * w with var the mean squared deviation (a layer norm
// with a weight and no bias).  S = 1 with mix = out = in = 1 is the ordinary residual sum x += y.  With ``rows``
// only those tokens are read and nothing is written back (the model's last norm at the wanted places); without
// ``in`` every stream counts once (the sum of the streams).  Streams, sums and statistics are float32.
#include "common.cuh"

constexpr int HC_MAX_STREAMS = 16;

// NS: the number of streams the loops are unrolled for (S <= NS)
template <typename TY, typename TO, int NS>
__global__ void __launch_bounds__(256, 4)
hc_norm_kernel(float* __restrict__ x, int64_t stream_stride, int S, const TY* __restrict__ y,
               const float* __restrict__ mix, const float* __restrict__ outw, const float* __restrict__ inw,
               const float* __restrict__ normw, float eps, TO* __restrict__ out, const int* __restrict__ rows, int W,
               const float* __restrict__ conv_w, float* __restrict__ conv_state, const int* __restrict__ state_slots,
               const int* __restrict__ context_lens, int taps) {
  extern __shared__ float u_s[];               // the token's u, W floats
  __shared__ float red[32];
  __shared__ float c_mix[HC_MAX_STREAMS * HC_MAX_STREAMS], c_out[HC_MAX_STREAMS], c_in[HC_MAX_STREAMS];
  const int tid = threadIdx.x;
  for (int i = tid; i < S * S; i += blockDim.x) c_mix[i] = mix ? mix[i] : 0.f;
  for (int i = tid; i < S; i += blockDim.x) {
    c_out[i] = outw ? outw[i] : 0.f;
    c_in[i] = inw ? inw[i] : 1.f;
  }
  pdl_wait();
  pdl_launch_dependents();
  __syncthreads();
  const int r_out = blockIdx.x;
  const int64_t t = rows ? rows[r_out] : r_out;
  float sum = 0.f;
  for (int w = tid; w < W; w += blockDim.x) {
    float xs[NS];
#pragma unroll
    for (int s = 0; s < NS; ++s)
      if (s < S) xs[s] = x[s * stream_stride + t * W + w];
    if (y != nullptr) {
      const float yy = to_f<TY>(y[t * W + w]);
      float nx[NS];
#pragma unroll
      for (int r = 0; r < NS; ++r) {
        if (r < S) {
          float a = 0.f;
#pragma unroll
          for (int s = 0; s < NS; ++s)
            if (s < S) a = fmaf(c_mix[s * S + r], xs[s], a);
          nx[r] = fmaf(c_out[r], yy, a);
        }
      }
#pragma unroll
      for (int r = 0; r < NS; ++r) {
        if (r < S) {
          xs[r] = nx[r];
          if (rows == nullptr) x[r * stream_stride + t * W + w] = nx[r];
        }
      }
    }
    float u = 0.f;
#pragma unroll
    for (int s = 0; s < NS; ++s)
      if (s < S) u = fmaf(c_in[s], xs[s], u);
    u_s[w] = u;
    sum += u;
  }
  if (normw == nullptr) return;                 // the update alone
  const float mean = block_sum(sum, red) / (float)W;
  float sq = 0.f;
  for (int w = tid; w < W; w += blockDim.x) {
    const float d = u_s[w] - mean;
    sq = fmaf(d, d, sq);
  }
  const float rstd = 1.0f / sqrtf(block_sum(sq, red) / (float)W + eps);
  if (conv_w == nullptr) {
    for (int w = tid; w < W; w += blockDim.x)
      out[(int64_t)r_out * W + w] = from_f<TO>((u_s[w] - mean) * rstd * normw[w]);
    return;
  }
  // Every request brings one token (token t is request t): the short convolution h + conv(h) of csrc/short_conv.cu
  // needs no other token of the step, only the request's state, which then moves up by one row and takes h.
  const int slot = state_slots[t], pos = context_lens[t] - 1;
  for (int w = tid; w < W; w += blockDim.x) {
    const float h = (u_s[w] - mean) * rstd * normw[w];
    float acc = h;
    if (slot >= 0 && taps > 1) {
      float* st = conv_state + (int64_t)slot * (taps - 1) * W + w;
      for (int j = 0; j < taps - 1; ++j) {
        const bool before_start = pos - (taps - 1) + j < 0;
        const float v = before_start ? 0.f : st[(int64_t)j * W];
        if (!before_start) acc = fmaf(conv_w[(int64_t)w * taps + j], v, acc);
        if (j > 0) st[(int64_t)(j - 1) * W] = v;
      }
      st[(int64_t)(taps - 2) * W] = h;
    }
    acc = fmaf(conv_w[(int64_t)w * taps + taps - 1], h, acc);
    out[(int64_t)r_out * W + w] = from_f<TO>(acc);
  }
}

template <typename TY, typename TO, int NS>
static int launch_hc_norm(float* x, int64_t stream_stride, int S, const void* y, const float* mix, const float* outw,
                          const float* inw, const float* normw, float eps, void* out, const int* rows, int n, int W, int threads,
                          size_t smem, const float* conv_w, float* conv_state, const int* state_slots, const int* context_lens,
                          int taps, cudaStream_t stream) {
  if (smem > 48 * 1024) {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(hc_norm_kernel<TY, TO, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      ME_REQUIRE(e == cudaSuccess, "me_hc_norm: cannot raise shared memory: %s", cudaGetErrorString(e));
      attr_set = true;
    }
  }
  me_launch(hc_norm_kernel<TY, TO, NS>, dim3(n), dim3(threads), smem, stream, x, stream_stride, S, (const TY*)y, mix, outw, inw,
            normw, eps, (TO*)out, rows, W, conv_w, conv_state, state_slots, context_lens, taps);
  return 0;
}

// x: [S, T, W] float32 (streams ``stream_stride`` elements apart).  y: [T, W] of y_dtype or null (no pending update;
// mix and outw are then unused).  inw: [S] or null (ones).  normw: [W] or null (no output).  out: [n, W] of out_dtype,
// n = number of rows if ``rows`` is given, else T.  conv_w [W, taps] (or null): every request brings one token, and the
// output is h + conv(h) with conv_state [slots, taps-1, W] renewed in place (state_slots and context_lens per request).
ME_API int me_hc_norm(float* x, int64_t stream_stride, int S, const void* y, int y_dtype, const float* mix,
                      const float* outw, const float* inw, const float* normw, float eps, void* out, int out_dtype,
                      const int* rows, int n, int W, const float* conv_w, float* conv_state, const int* state_slots,
                      const int* context_lens, int taps, cudaStream_t stream) {
  if (n == 0) return 0;
  ME_REQUIRE(S >= 1 && S <= HC_MAX_STREAMS, "me_hc_norm: %d streams (1 to %d are supported)", S, HC_MAX_STREAMS);
  ME_REQUIRE(n > 0 && W > 0, "me_hc_norm: bad sizes n=%d W=%d", n, W);
  ME_REQUIRE(y == nullptr || (mix != nullptr && outw != nullptr), "me_hc_norm: an update needs mix and out weights");
  ME_REQUIRE(normw == nullptr || out != nullptr, "me_hc_norm: a norm needs an output");
  ME_REQUIRE(conv_w == nullptr || (rows == nullptr && normw != nullptr && taps >= 1 && state_slots != nullptr && context_lens != nullptr
                                   && (taps == 1 || conv_state != nullptr)),
             "me_hc_norm: the convolution needs a norm, all rows, the requests' slots and lengths, and a state");
  const size_t smem = sizeof(float) * (size_t)W;
  ME_REQUIRE(smem <= 160 * 1024, "me_hc_norm: width %d is too large", W);
  const int threads = W >= 1024 ? 256 : (W >= 256 ? 128 : 64);
  int rc = 0;
  ME_DISPATCH_DTYPE(y_dtype, TY, ME_DISPATCH_DTYPE(out_dtype, TO, {
    if (S == 1) rc = launch_hc_norm<TY, TO, 1>(x, stream_stride, S, y, mix, outw, inw, normw, eps, out, rows, n, W, threads, smem, conv_w, conv_state, state_slots, context_lens, taps, stream);
    else if (S == 2) rc = launch_hc_norm<TY, TO, 2>(x, stream_stride, S, y, mix, outw, inw, normw, eps, out, rows, n, W, threads, smem, conv_w, conv_state, state_slots, context_lens, taps, stream);
    else if (S <= 4) rc = launch_hc_norm<TY, TO, 4>(x, stream_stride, S, y, mix, outw, inw, normw, eps, out, rows, n, W, threads, smem, conv_w, conv_state, state_slots, context_lens, taps, stream);
    else if (S <= 8) rc = launch_hc_norm<TY, TO, 8>(x, stream_stride, S, y, mix, outw, inw, normw, eps, out, rows, n, W, threads, smem, conv_w, conv_state, state_slots, context_lens, taps, stream);
    else rc = launch_hc_norm<TY, TO, HC_MAX_STREAMS>(x, stream_stride, S, y, mix, outw, inw, normw, eps, out, rows, n, W, threads, smem, conv_w, conv_state, state_slots, context_lens, taps, stream);
  }));
  if (rc) return rc;
  ME_LAUNCH_CHECK("me_hc_norm");
  return 0;
}
