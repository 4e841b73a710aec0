// The norm kernel of blocks that normalise a sub-layer's output before it joins the residual stream:
//
//   x <- x + mult * y / rms(y) * post_w          (y: a sub-layer's output, post_w: the weight of the norm behind it)
//   out = x / rms(x) * pre_w                      (the norm in front of the next sub-layer; pre_w absent: out = x)
//
// rms(v) = sqrt(mean(v^2) + eps) with one eps for both.  The residual stream x is float32 [T, W]; sums, statistics and
// weights are float32 and a row's sums are taken in a fixed order.  With ``rows`` only those rows are read and x is
// left as it is (the model's last norm at the places whose logits are wanted).  Either half may be absent.
#include "common.cuh"

// Four neighbouring elements at once where the rows allow it (W a multiple of 4 and 16-byte aligned tensors).
template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<bf16>(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&lo);
  raw.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TY, typename TO, int VEC>
__global__ void __launch_bounds__(256)
sandwich_norm_kernel(float* __restrict__ x, const TY* __restrict__ y, const float* __restrict__ post_w, float mult,
                     const float* __restrict__ pre_w, float eps, TO* __restrict__ out, const int* __restrict__ rows, int W,
                     int norm_out) {
  extern __shared__ __align__(16) float row[];
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
    for (int i = threadIdx.x * VEC; i < W; i += blockDim.x * VEC) {
      if (VEC == 4) {
        const float4 v = load4<TY>(yr + i);
        *reinterpret_cast<float4*>(row + i) = v;
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
      } else {
        const float v = to_f<TY>(yr[i]);
        row[i] = v;
        ss = fmaf(v, v, ss);
      }
    }
    ry = rsqrtf(block_sum(ss, red) * inv_w + eps) * mult;
  }
  float ss = 0.f;
  for (int i = threadIdx.x * VEC; i < W; i += blockDim.x * VEC) {
    if (VEC == 4) {
      float4 v = *reinterpret_cast<const float4*>(xr + i);
      if (y) {
        const float4 u = *reinterpret_cast<const float4*>(row + i), w = *reinterpret_cast<const float4*>(post_w + i);
        v.x = fmaf(u.x * ry, w.x, v.x);
        v.y = fmaf(u.y * ry, w.y, v.y);
        v.z = fmaf(u.z * ry, w.z, v.z);
        v.w = fmaf(u.w * ry, w.w, v.w);
        if (!rows) *reinterpret_cast<float4*>(xr + i) = v;
      }
      *reinterpret_cast<float4*>(row + i) = v;
      ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    } else {
      float v = xr[i];
      if (y) {
        v = fmaf(row[i] * ry, post_w[i], v);
        if (!rows) xr[i] = v;
      }
      row[i] = v;
      ss = fmaf(v, v, ss);
    }
  }
  if (!out) return;
  TO* o = out + (int64_t)blockIdx.x * W;
  const float rx = norm_out ? rsqrtf(block_sum(ss, red) * inv_w + eps) : 1.f;     // (a thread reads back what it wrote itself)
  for (int i = threadIdx.x * VEC; i < W; i += blockDim.x * VEC) {
    if (VEC == 4) {
      float4 v = *reinterpret_cast<const float4*>(row + i);
      if (norm_out) {
        const float4 w = pre_w ? *reinterpret_cast<const float4*>(pre_w + i) : make_float4(1.f, 1.f, 1.f, 1.f);
        v = make_float4(v.x * rx * w.x, v.y * rx * w.y, v.z * rx * w.z, v.w * rx * w.w);
      }
      store4(o + i, v);
    } else {
      o[i] = from_f<TO>(norm_out ? row[i] * rx * (pre_w ? pre_w[i] : 1.f) : row[i]);
    }
  }
}

// x: [T, W] float32.  y: [T, W] of y_dtype or null.  post_w, pre_w: [W] float32 or null.  out: [n, W] of out_dtype or null.
// rows: [n] int32 or null (then n == T).  norm_out == 0: out is x itself, not normalised.
ME_API int me_sandwich_norm(float* x, const void* y, int y_dtype, const float* post_w, float mult, const float* pre_w, float eps,
                            void* out, int out_dtype, const int* rows, int n, int W, int norm_out, cudaStream_t stream) {
  if (n == 0) return 0;
  ME_REQUIRE(n > 0 && W > 0 && W <= 24576, "me_sandwich_norm: bad sizes n=%d W=%d", n, W);
  ME_REQUIRE(!y || post_w, "me_sandwich_norm: an output to add needs the weight of its norm");
  const int threads = W >= 2048 ? 256 : (W >= 512 ? 128 : 64);
  const size_t smem = sizeof(float) * W;
  const auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const bool vec = W % 4 == 0 && aligned(x) && aligned(y) && aligned(post_w) && aligned(pre_w) && aligned(out);
  ME_DISPATCH_DTYPE(y ? y_dtype : ME_F32, TY, ME_DISPATCH_DTYPE(out ? out_dtype : ME_F32, TO, {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e1 = cudaFuncSetAttribute(sandwich_norm_kernel<TY, TO, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      cudaError_t e4 = cudaFuncSetAttribute(sandwich_norm_kernel<TY, TO, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      ME_REQUIRE(e1 == cudaSuccess && e4 == cudaSuccess, "me_sandwich_norm: cannot raise shared memory");
      attr_set = true;
    }
    if (vec)
      me_launch(sandwich_norm_kernel<TY, TO, 4>, dim3(n), dim3(threads), smem, stream, x, (const TY*)y, post_w, mult, pre_w, eps,
                (TO*)out, rows, W, norm_out);
    else
      me_launch(sandwich_norm_kernel<TY, TO, 1>, dim3(n), dim3(threads), smem, stream, x, (const TY*)y, post_w, mult, pre_w, eps,
                (TO*)out, rows, W, norm_out);
  }));
  ME_LAUNCH_CHECK("me_sandwich_norm");
  return 0;
}
