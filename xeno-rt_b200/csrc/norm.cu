// RMSNorm over rows of the 32-bit residual stream: y = (x * rsqrt(mean(x^2) + eps)) * w.
// Restates crates/xrt-kernels/src/cpu/rmsnorm.rs:26-43 and the reference's PTX rmsnorm_kernel
// (crates/xrt-cuda/src/lib.rs:41-224: one block a row, a tree reduction, then the scaling).
// Statistics are 32-bit; the output is 32-bit or bfloat16.  With `rows` the kernel gathers:
// output row r is the norm of input row rows[r] (used for the rows whose logits are wanted).
//
// A decode step normalises a handful of rows, so the kernel's time is load latency, not
// bandwidth: a row is read once with 16-byte loads that are all issued before the first is used
// (up to eight a thread, kept in registers for the scaling pass), one block a row.
#include "common.cuh"

namespace xrt {

constexpr int NORM_THREADS = 256;

template <typename TW> struct Vec4Of;
template <> struct Vec4Of<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
};
template <> struct Vec4Of<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
  }
};
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&a);
  t.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

// width is a multiple of 4 and at most CHUNKS * NORM_THREADS * 4
template <typename TW, typename TO, int CHUNKS>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_vec_kernel(TO* __restrict__ out, const float* __restrict__ x, const TW* __restrict__ w,
                   const int* __restrict__ rows, int width, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  // the weight does not depend on the step: it is on its way while the kernel before this one finishes
  float wv[CHUNKS][4];
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (threadIdx.x + i * NORM_THREADS) * 4;
    if (c < width) Vec4Of<TW>::load(w + c, wv[i]);
  }
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows != nullptr ? rows[r] : r;
  const float* xr = x + (size_t)src * width;
  float v[CHUNKS][4];
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (threadIdx.x + i * NORM_THREADS) * 4;
    if (c < width) Vec4Of<float>::load(xr + c, v[i]);
    else v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
  }
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc = fmaf(v[i][j], v[i][j], acc);
  const float total = block_sum(acc, scratch);
  const float inv = 1.0f / sqrtf(total / (float)width + eps);
  TO* dst = out + (size_t)r * width;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (threadIdx.x + i * NORM_THREADS) * 4;
    if (c < width) {
      float y[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) y[j] = (v[i][j] * inv) * wv[i][j];
      store4(dst + c, y);
    }
  }
}

// any width
template <typename TW, typename TO>
__global__ void rmsnorm_kernel(TO* __restrict__ out, const float* __restrict__ x, const TW* __restrict__ w,
                               const int* __restrict__ rows, int width, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows != nullptr ? rows[r] : r;
  const float* xr = x + (size_t)src * width;
  float acc = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = xr[c];
    acc = fmaf(v, v, acc);
  }
  const float total = block_sum(acc, scratch);
  const float inv = 1.0f / sqrtf(total / (float)width + eps);
  TO* dst = out + (size_t)r * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    dst[c] = from_float<TO>((xr[c] * inv) * to_float(w[c]));
}

// Layer norm with a weight and no bias: y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * w, any width.
// Two sums over the row in a fixed order (the mean first, then the squared deviations from it).
// width is a multiple of 4 and at most CHUNKS * NORM_THREADS * 4: the row stays in registers, read once with
// 16-byte loads that are all in flight together (as rmsnorm_vec_kernel does)
template <typename TW, typename TO, int CHUNKS>
__global__ void __launch_bounds__(NORM_THREADS)
layernorm_vec_kernel(TO* __restrict__ out, const float* __restrict__ x, const TW* __restrict__ w,
                     const int* __restrict__ rows, int width, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  float wv[CHUNKS][4];
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (threadIdx.x + i * NORM_THREADS) * 4;
    if (c < width) Vec4Of<TW>::load(w + c, wv[i]);
  }
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows != nullptr ? rows[r] : r;
  const float* xr = x + (size_t)src * width;
  float v[CHUNKS][4];
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (threadIdx.x + i * NORM_THREADS) * 4;
    if (c < width) Vec4Of<float>::load(xr + c, v[i]);
    else v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
  }
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc += v[i][j];
  const float mean = block_sum(acc, scratch) / (float)width;
  acc = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (threadIdx.x + i * NORM_THREADS) * 4;
    if (c < width) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[i][j] -= mean;
        acc = fmaf(v[i][j], v[i][j], acc);
      }
    }
  }
  const float inv = 1.0f / sqrtf(block_sum(acc, scratch) / (float)width + eps);
  TO* dst = out + (size_t)r * width;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (threadIdx.x + i * NORM_THREADS) * 4;
    if (c < width) {
      float y[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) y[j] = (v[i][j] * inv) * wv[i][j];
      store4(dst + c, y);
    }
  }
}

template <typename TW, typename TO>
__global__ void layernorm_kernel(TO* __restrict__ out, const float* __restrict__ x, const TW* __restrict__ w,
                                 const int* __restrict__ rows, int width, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows != nullptr ? rows[r] : r;
  const float* xr = x + (size_t)src * width;
  float acc = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) acc += xr[c];
  const float mean = block_sum(acc, scratch) / (float)width;
  acc = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float d = xr[c] - mean;
    acc = fmaf(d, d, acc);
  }
  const float inv = 1.0f / sqrtf(block_sum(acc, scratch) / (float)width + eps);
  TO* dst = out + (size_t)r * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    dst[c] = from_float<TO>(((xr[c] - mean) * inv) * to_float(w[c]));
}

// Layer norm with a weight and an optional bias over the sum of `n_parts` inputs (x + p * part_stride, added in index
// order), y = (x - mean) / sqrt(var + eps) * w + b.  With `residual` the result is added to that 32-bit row instead of
// written to `out`: a norm that follows a sublayer, and the residual sum, in one pass; with `residual` AND `out` the
// new residual row is then normed again with (w2, b2) into `out`: the norm that the next sublayer begins with.
// The row is kept in shared memory.
// Sum over the block with one barrier: lanes by butterfly, then every thread adds the warps' sums in index order.
// `scratch` is one of two arrays of 32 floats used in turn, so that a sum may begin while slow threads still read
// the one before.
__device__ __forceinline__ float block_sum_once(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < n_warps; ++w) total += scratch[w];
  return total;
}

template <typename TO>
__global__ void layernorm_affine_kernel(TO* __restrict__ out, float* __restrict__ residual, const float* __restrict__ x,
                                        int n_parts, size_t part_stride, const float* __restrict__ w,
                                        const float* __restrict__ b, const int* __restrict__ rows, int width, float eps,
                                        const float* __restrict__ w2, const float* __restrict__ b2) {
  extern __shared__ float row[];
  __shared__ float scratch[4][32];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows != nullptr ? rows[r] : r;
  const float* xr = x + (size_t)src * width;
  float acc = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = xr[c];
    for (int p = 1; p < n_parts; ++p) v += xr[p * part_stride + c];
    row[c] = v;
    acc += v;
  }
  float mean = block_sum_once(acc, scratch[0]) / (float)width;
  acc = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float d = row[c] - mean;
    acc = fmaf(d, d, acc);
  }
  float inv = 1.0f / sqrtf(block_sum_once(acc, scratch[1]) / (float)width + eps);
  acc = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float y = ((row[c] - mean) * inv) * w[c] + (b != nullptr ? b[c] : 0.f);
    if (residual != nullptr) {
      const float sum = residual[(size_t)r * width + c] + y;
      residual[(size_t)r * width + c] = sum;
      row[c] = sum;  // a thread reads back only what it wrote
      acc += sum;
    } else {
      out[(size_t)r * width + c] = from_float<TO>(y);
    }
  }
  if (residual == nullptr || out == nullptr) return;
  mean = block_sum_once(acc, scratch[2]) / (float)width;
  acc = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float d = row[c] - mean;
    acc = fmaf(d, d, acc);
  }
  inv = 1.0f / sqrtf(block_sum_once(acc, scratch[3]) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[(size_t)r * width + c] = from_float<TO>(((row[c] - mean) * inv) * w2[c] + (b2 != nullptr ? b2[c] : 0.f));
}

// The same for rows of up to 256 * ITEMS floats, held in registers: the weights and biases of both norms are asked
// for before the wait for the kernel before, the row and the residual together after it, so that a row of a decode
// step costs two trips to memory instead of six in a row.
template <typename TO, int ITEMS>
__global__ void __launch_bounds__(256)
layernorm_affine_rows_kernel(TO* __restrict__ out, float* __restrict__ residual, const float* __restrict__ x, int n_parts,
                             size_t part_stride, const float* __restrict__ w, const float* __restrict__ b,
                             const int* __restrict__ rows, int width, float eps, const float* __restrict__ w2,
                             const float* __restrict__ b2) {
  __shared__ float scratch[4][32];
  pdl_trigger();
  float wv[ITEMS], bv[ITEMS], w2v[ITEMS], b2v[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int c = threadIdx.x + i * 256;
    const bool in = c < width;
    wv[i] = in ? w[c] : 0.f;
    bv[i] = in && b != nullptr ? b[c] : 0.f;
    w2v[i] = in && w2 != nullptr ? w2[c] : 0.f;
    b2v[i] = in && b2 != nullptr ? b2[c] : 0.f;
  }
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows != nullptr ? rows[r] : r;
  const float* xr = x + (size_t)src * width;
  float v[ITEMS], res[ITEMS];
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int c = threadIdx.x + i * 256;
    v[i] = 0.f;
    res[i] = 0.f;
    if (c < width) {
      v[i] = xr[c];
      for (int p = 1; p < n_parts; ++p) v[i] += xr[p * part_stride + c];
      if (residual != nullptr) res[i] = residual[(size_t)r * width + c];
    }
    acc += v[i];
  }
  float mean = block_sum_once(acc, scratch[0]) / (float)width;
  acc = 0.f;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const float d = threadIdx.x + i * 256 < width ? v[i] - mean : 0.f;
    acc = fmaf(d, d, acc);
  }
  float inv = 1.0f / sqrtf(block_sum_once(acc, scratch[1]) / (float)width + eps);
  acc = 0.f;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < width) {
      const float y = ((v[i] - mean) * inv) * wv[i] + bv[i];
      if (residual != nullptr) {
        v[i] = res[i] + y;
        residual[(size_t)r * width + c] = v[i];
        acc += v[i];
      } else {
        out[(size_t)r * width + c] = from_float<TO>(y);
      }
    }
  }
  if (residual == nullptr || out == nullptr) return;
  mean = block_sum_once(acc, scratch[2]) / (float)width;
  acc = 0.f;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const float d = threadIdx.x + i * 256 < width ? v[i] - mean : 0.f;
    acc = fmaf(d, d, acc);
  }
  inv = 1.0f / sqrtf(block_sum_once(acc, scratch[3]) / (float)width + eps);
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < width) out[(size_t)r * width + c] = from_float<TO>(((v[i] - mean) * inv) * w2v[i] + b2v[i]);
  }
}

}  // namespace xrt

XRT_EXPORT int xrt_layernorm_affine(void* out, float* residual, const float* x, int n_parts, long long part_stride,
                                    const float* weight, const float* bias, const int* rows, int n_rows, int width,
                                    float eps, int out_dtype, const float* weight2, const float* bias2,
                                    cudaStream_t stream) {
  if (n_rows < 0 || width <= 0 || n_parts < 1 || (out == nullptr && residual == nullptr)) return XRT_ERR_ARGUMENT;
  if (out != nullptr && residual != nullptr && (weight2 == nullptr || rows != nullptr)) return XRT_ERR_ARGUMENT;
  if ((size_t)width * sizeof(float) > 160 * 1024) return XRT_ERR_UNSUPPORTED;
  if (n_rows == 0) return XRT_OK;
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
  const size_t smem = (size_t)width * sizeof(float);
  if (width <= 256 * 16) {
    XRT_DISPATCH_DTYPE(out_dtype, TO, {
      if (width <= 256 * 4)
        xrt::launch_kernel(xrt::layernorm_affine_rows_kernel<TO, 4>, dim3(n_rows), dim3(256), 0, stream, (TO*)out, residual, x,
                           n_parts, (size_t)part_stride, weight, bias, rows, width, eps, weight2, bias2);
      else if (width <= 256 * 8)
        xrt::launch_kernel(xrt::layernorm_affine_rows_kernel<TO, 8>, dim3(n_rows), dim3(256), 0, stream, (TO*)out, residual, x,
                           n_parts, (size_t)part_stride, weight, bias, rows, width, eps, weight2, bias2);
      else
        xrt::launch_kernel(xrt::layernorm_affine_rows_kernel<TO, 16>, dim3(n_rows), dim3(256), 0, stream, (TO*)out, residual, x,
                           n_parts, (size_t)part_stride, weight, bias, rows, width, eps, weight2, bias2);
    });
    return xrt::launch_status();
  }
  XRT_DISPATCH_DTYPE(out_dtype, TO, {
    auto kernel = xrt::layernorm_affine_kernel<TO>;
    if (smem > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return (int)err;
    }
    xrt::launch_kernel(kernel, dim3(n_rows), dim3(threads), smem, stream, (TO*)out, residual, x, n_parts,
                       (size_t)part_stride, weight, bias, rows, width, eps, weight2, bias2);
  });
  return xrt::launch_status();
}


XRT_EXPORT int xrt_layernorm(void* out, const float* x, const void* weight, const int* rows, int n_rows,
                             int width, float eps, int weight_dtype, int out_dtype, cudaStream_t stream) {
  if (n_rows < 0 || width <= 0) return XRT_ERR_ARGUMENT;
  if (n_rows == 0) return XRT_OK;
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
  const bool vec = width % 4 == 0 && (((uintptr_t)x | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
  const int chunks = (width / 4 + xrt::NORM_THREADS - 1) / xrt::NORM_THREADS;
  XRT_DISPATCH_DTYPE(weight_dtype, TW, {
    XRT_DISPATCH_DTYPE(out_dtype, TO, {
      if (vec && chunks <= 1)
        xrt::launch_kernel(xrt::layernorm_vec_kernel<TW, TO, 1>, dim3(n_rows), dim3(xrt::NORM_THREADS), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
      else if (vec && chunks <= 2)
        xrt::launch_kernel(xrt::layernorm_vec_kernel<TW, TO, 2>, dim3(n_rows), dim3(xrt::NORM_THREADS), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
      else if (vec && chunks <= 4)
        xrt::launch_kernel(xrt::layernorm_vec_kernel<TW, TO, 4>, dim3(n_rows), dim3(xrt::NORM_THREADS), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
      else if (vec && chunks <= 8)
        xrt::launch_kernel(xrt::layernorm_vec_kernel<TW, TO, 8>, dim3(n_rows), dim3(xrt::NORM_THREADS), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
      else
        xrt::launch_kernel(xrt::layernorm_kernel<TW, TO>, dim3(n_rows), dim3(threads), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
    });
  });
  return xrt::launch_status();
}

XRT_EXPORT int xrt_rmsnorm(void* out, const float* x, const void* weight, const int* rows, int n_rows,
                           int width, float eps, int weight_dtype, int out_dtype, cudaStream_t stream) {
  if (n_rows < 0 || width <= 0) return XRT_ERR_ARGUMENT;
  if (n_rows == 0) return XRT_OK;
  const bool vec = width % 4 == 0 && width <= 8 * xrt::NORM_THREADS * 4 && (((uintptr_t)x | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
  const int chunks = (width / 4 + xrt::NORM_THREADS - 1) / xrt::NORM_THREADS;
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
  XRT_DISPATCH_DTYPE(weight_dtype, TW, {
    XRT_DISPATCH_DTYPE(out_dtype, TO, {
      if (vec && chunks <= 1)
        xrt::launch_kernel(xrt::rmsnorm_vec_kernel<TW, TO, 1>, dim3(n_rows), dim3(xrt::NORM_THREADS), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
      else if (vec && chunks <= 2)
        xrt::launch_kernel(xrt::rmsnorm_vec_kernel<TW, TO, 2>, dim3(n_rows), dim3(xrt::NORM_THREADS), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
      else if (vec && chunks <= 4)
        xrt::launch_kernel(xrt::rmsnorm_vec_kernel<TW, TO, 4>, dim3(n_rows), dim3(xrt::NORM_THREADS), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
      else if (vec)
        xrt::launch_kernel(xrt::rmsnorm_vec_kernel<TW, TO, 8>, dim3(n_rows), dim3(xrt::NORM_THREADS), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
      else
        xrt::launch_kernel(xrt::rmsnorm_kernel<TW, TO>, dim3(n_rows), dim3(threads), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
    });
  });
  return xrt::launch_status();
}
