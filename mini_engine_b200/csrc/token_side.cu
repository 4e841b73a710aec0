// The middle of a layer's token input: g[t, j] = gelu_tanh(z[t, j]) * table[token_t, first + j], where z is the product of
// the stream with the layer's gate matrix and ``table`` a second embedding of which every layer has a slice of ``dim``
// columns.  gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).  A token id ~j stands for feedback[j].
#include "common.cuh"

template <typename TZ, typename TE, typename TO>
__global__ void __launch_bounds__(128)
token_side_gate_kernel(const TZ* __restrict__ z, int64_t z_stride, const int* __restrict__ ids, const int* __restrict__ feedback,
                       const TE* __restrict__ table, int64_t table_stride, int vocab, int first, int dim, TO* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && feedback) id = feedback[~id];
  if (id < 0 || id >= vocab) id = 0;           // the embedding kernel has flagged it
  for (int j = threadIdx.x; j < dim; j += blockDim.x) {
    const float v = to_f<TZ>(z[(int64_t)t * z_stride + j]);
    const float gelu = 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    out[(int64_t)t * dim + j] = from_f<TO>(gelu * to_f<TE>(table[(int64_t)id * table_stride + first + j]));
  }
}

ME_API int me_token_side_gate(const void* z, int z_dtype, int64_t z_stride, const int* ids, const int* feedback, const void* table,
                              int table_dtype, int64_t table_stride, int vocab, int first, int dim, void* out, int out_dtype, int T,
                              cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(dim > 0 && first >= 0 && first + dim <= table_stride, "me_token_side_gate: slice [%d, %d) of %lld columns", first,
             first + dim, (long long)table_stride);
  ME_DISPATCH_DTYPE(z_dtype, TZ, ME_DISPATCH_DTYPE(table_dtype, TE, ME_DISPATCH_DTYPE(out_dtype, TO,
      me_launch(token_side_gate_kernel<TZ, TE, TO>, dim3(T), dim3(128), 0, stream, (const TZ*)z, z_stride, ids, feedback,
                (const TE*)table, table_stride, vocab, first, dim, (TO*)out))));
  ME_LAUNCH_CHECK("me_token_side_gate");
  return 0;
}

// The whole token input of a layer for a step of few tokens, in one kernel (a decode step is a chain of short kernels: this
// one stands for four): the pending update of the stream x <- x + mult * y / rms(y) * post_w, then z = W_gate x,
// g = gelu_tanh(z) * table[token, first + j], out = W_proj g.  A block a token: the stream's row in shared memory, a warp a
// few of the ``dim`` gate rows, a thread a few of the output's elements.  In the bfloat16 engine x and g are rounded to
// bfloat16 before their products, as the separate kernels round them.
template <typename TY, typename TW, typename TE, typename TO>
__global__ void __launch_bounds__(256)
token_side_fused_kernel(float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ post_w, float mult, float eps,
                        const TW* __restrict__ w_gate, const TW* __restrict__ w_proj, const int* __restrict__ ids,
                        const int* __restrict__ feedback, const TE* __restrict__ table, int64_t table_stride, int vocab, int first,
                        int dim, TO* __restrict__ out, int W) {
  extern __shared__ float ts_smem[];                 // [W] the stream's row, [dim] g
  __shared__ float red[32];
  float* xs = ts_smem;
  float* gs = ts_smem + W;
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  float* xr = x + (int64_t)t * W;
  float ry = 0.f;
  if (y) {
    const TY* yr = y + (int64_t)t * W;
    float ss = 0.f;
    for (int i = tid; i < W; i += blockDim.x) {
      const float v = to_f<TY>(yr[i]);
      xs[i] = v;
      ss = fmaf(v, v, ss);
    }
    ry = rsqrtf(block_sum(ss, red) / (float)W + eps) * mult;
  }
  for (int i = tid; i < W; i += blockDim.x) {
    float v = xr[i];
    if (y) {
      v = fmaf(xs[i] * ry, post_w[i], v);
      xr[i] = v;
    }
    xs[i] = to_f<TO>(from_f<TO>(v));                 // what the gate's product reads: the stream in the working dtype
  }
  __syncthreads();
  int id = ids[t];
  if (id < 0 && feedback) id = feedback[~id];
  if (id < 0 || id >= vocab) id = 0;                 // the embedding kernel has flagged it
  for (int j = warp; j < dim; j += nwarps) {
    const TW* wr = w_gate + (int64_t)j * W;
    float acc = 0.f;
    for (int i = lane; i < W; i += 32) acc = fmaf(to_f<TW>(wr[i]), xs[i], acc);
    acc = warp_sum(acc);
    if (lane == 0) {
      const float gelu = 0.5f * acc * (1.f + tanhf(0.7978845608028654f * (acc + 0.044715f * acc * acc * acc)));
      gs[j] = to_f<TO>(from_f<TO>(gelu * to_f<TE>(table[(int64_t)id * table_stride + first + j])));
    }
  }
  __syncthreads();
  for (int i = tid; i < W; i += blockDim.x) {
    const TW* wr = w_proj + (int64_t)i * dim;
    float acc = 0.f;
    for (int j = 0; j < dim; ++j) acc = fmaf(to_f<TW>(wr[j]), gs[j], acc);
    out[(int64_t)t * W + i] = from_f<TO>(acc);
  }
}

// x: [T, W] float32 (updated in place when y is given).  y: [T, W] of y_dtype or null, post_w [W] float32.  w_gate: [dim, W],
// w_proj: [W, dim] of w_dtype.  out: [T, W] of out_dtype, which is also the working dtype x and g are rounded to.
ME_API int me_token_side_fused(float* x, const void* y, int y_dtype, const float* post_w, float mult, float eps, const void* w_gate,
                               const void* w_proj, int w_dtype, const int* ids, const int* feedback, const void* table,
                               int table_dtype, int64_t table_stride, int vocab, int first, int dim, void* out, int out_dtype, int T,
                               int W, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(dim > 0 && first >= 0 && first + dim <= table_stride && W > 0 && (W + dim) * 4 <= 96 * 1024, "me_token_side_fused: bad sizes");
  ME_REQUIRE(!y || post_w, "me_token_side_fused: an output to add needs the weight of its norm");
  const size_t smem = sizeof(float) * (W + dim);
  ME_DISPATCH_DTYPE(y ? y_dtype : ME_F32, TY, ME_DISPATCH_DTYPE(w_dtype, TW, ME_DISPATCH_DTYPE(table_dtype, TE, ME_DISPATCH_DTYPE(out_dtype, TO, {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(token_side_fused_kernel<TY, TW, TE, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      ME_REQUIRE(e == cudaSuccess, "me_token_side_fused: cannot raise shared memory: %s", cudaGetErrorString(e));
      attr_set = true;
    }
    me_launch(token_side_fused_kernel<TY, TW, TE, TO>, dim3(T), dim3(256), smem, stream, x, (const TY*)y, post_w, mult, eps,
              (const TW*)w_gate, (const TW*)w_proj, ids, feedback, (const TE*)table, table_stride, vocab, first, dim, (TO*)out, W);
  }))));
  ME_LAUNCH_CHECK("me_token_side_fused");
  return 0;
}
