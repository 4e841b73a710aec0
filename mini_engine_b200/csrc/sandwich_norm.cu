// The norm kernel of blocks that normalise a sub-layer's output before it joins the residual stream:
//
//   x <- x + mult * y / rms(y) * post_w          (y: a sub-layer's output, post_w: the weight of the norm behind it)
//   out = x / rms(x) * pre_w                      (the norm in front of the next sub-layer; pre_w absent: out = x)
//
// rms(v) = sqrt(mean(v^2) + eps) with one eps for both.  The residual stream x is float32 [T, W]; sums, statistics and
// weights are float32 and a row's sums are taken in a fixed order.  With ``rows`` only those rows are read and x is
// left as it is (the model's last norm at the places whose logits are wanted).  Either half may be absent.
#include "common.cuh"

template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
sandwich_norm_kernel(float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ post_w, float mult,
                     const float* __restrict__ pre_w, float eps, TO* __restrict__ out, const int* __restrict__ rows, int W,
                     int norm_out) {
  extern __shared__ float row[];
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* xr = x + (int64_t)r * W;
  const float inv_w = 1.0f / (float)W;
  float ry = 0.f;
  if (y) {
    const TY* yr = y + (int64_t)r * W;
    float ss = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float v = to_f<TY>(yr[i]);
      row[i] = v;
      ss = fmaf(v, v, ss);
    }
    ry = rsqrtf(block_sum(ss, red) * inv_w + eps) * mult;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = xr[i];
    if (y) {
      v = fmaf(row[i] * ry, post_w[i], v);
      if (!rows) xr[i] = v;
    }
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  if (!out) return;
  if (!norm_out) {
    for (int i = threadIdx.x; i < W; i += blockDim.x) out[(int64_t)blockIdx.x * W + i] = from_f<TO>(row[i]);
    return;
  }
  const float rx = rsqrtf(block_sum(ss, red) * inv_w + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x)
    out[(int64_t)blockIdx.x * W + i] = from_f<TO>(row[i] * rx * (pre_w ? pre_w[i] : 1.f));
}

// x: [T, W] float32.  y: [T, W] of y_dtype or null.  post_w, pre_w: [W] float32 or null.  out: [n, W] of out_dtype or null.
// rows: [n] int32 or null (then n == T).  norm_out == 0: out is x itself, not normalised.
ME_API int me_sandwich_norm(float* x, const void* y, int y_dtype, const float* post_w, float mult, const float* pre_w, float eps,
                            void* out, int out_dtype, const int* rows, int n, int W, int norm_out, cudaStream_t stream) {
  if (n == 0) return 0;
  ME_REQUIRE(n > 0 && W > 0 && W <= 24576, "me_sandwich_norm: bad sizes n=%d W=%d", n, W);
  ME_REQUIRE(!y || post_w, "me_sandwich_norm: an output to add needs the weight of its norm");
  const int threads = W >= 1024 ? 256 : (W >= 256 ? 128 : 64);
  const size_t smem = sizeof(float) * W;
  ME_DISPATCH_DTYPE(y ? y_dtype : ME_F32, TY, ME_DISPATCH_DTYPE(out ? out_dtype : ME_F32, TO, {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(sandwich_norm_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      ME_REQUIRE(e == cudaSuccess, "me_sandwich_norm: cannot raise shared memory: %s", cudaGetErrorString(e));
      attr_set = true;
    }
    me_launch(sandwich_norm_kernel<TY, TO>, dim3(n), dim3(threads), smem, stream, x, (const TY*)y, post_w, mult, pre_w, eps,
              (TO*)out, rows, W, norm_out);
  }));
  ME_LAUNCH_CHECK("me_sandwich_norm");
  return 0;
}
