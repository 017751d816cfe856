// A state-space recurrence with ONE scalar decay per head and token (the "state-space duality" form), and the
// gated group norm that follows it.  Everything here is 32-bit: step sizes, decays, the state, the norm.
//
//   step size   dt_t = softplus(raw_t + dt_bias[h])                      (no clamp)
//   scan        S_t = exp(-exp(a_log[h]) dt_t) S_(t-1) + dt_t b_t x_t^T,   y_t = S_t^T c_t + d_skip[h] x_t
//               S is [state, vdim] per head; b and c belong to the head's group (n_heads / n_groups heads share them)
//   group norm  v = y * silu(z); every one of `groups` equal stretches of the row is divided by its own root mean
//               square; times a weight
//
// A sequence is a row of the step's cu_seqlens / seq_slot arrays; a row with slot -1 or no tokens is skipped, so
// padding rows of a captured step leave every state alone.  The state is kept [slot][head][vdim][state]: a column
// of S is contiguous.  A token's arithmetic is the same whether it comes alone or inside a prompt, so results do
// not depend on how a sequence was cut into steps.
#include "common.cuh"

namespace xrt {

struct SsdArgs {
  float* out;                       // [T, heads * vdim]
  const float *x, *b, *c, *dt;      // rows of x_stride / bc_stride / dt_stride floats
  int x_stride, bc_stride, dt_stride;
  const float *dt_bias, *a_log, *d_skip;  // [heads]
  float* state;                     // [slots, heads, vdim, state]
  const int *cu_seqlens, *seq_slot;
  int n_heads, heads_per_group, n_state, vdim;
  int parts, cols, tile_tokens;
};

// One block: one sequence, one head, `cols` value columns.  A column's state (n_state rows) is held in registers by
// `parts` neighbouring lanes, R rows each (lane p holds rows p R .. p R + R - 1; rows beyond n_state stay zero);
// the read-out's sum over rows is finished by a butterfly among those lanes, so its order is fixed.  Tiles of
// `tile_tokens` tokens' b, c, x, step size and decay are staged in shared memory.
template <int R>
__global__ void __launch_bounds__(128) ssd_scan_kernel(const SsdArgs a) {
  extern __shared__ __align__(16) float tile[];
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y;
  const int slot = a.seq_slot[s];
  const int begin = a.cu_seqlens[s], end = a.cu_seqlens[s + 1];
  if (slot < 0 || end <= begin) return;
  const int parts = a.parts, cols = a.cols, TT = a.tile_tokens, n_state = a.n_state, vdim = a.vdim;
  const int padded = parts * R;
  const int part = threadIdx.x % parts, jl = threadIdx.x / parts;
  const int col0 = blockIdx.z * cols, j = col0 + jl;
  const int g = h / a.heads_per_group;
  const bool live = j < vdim;
  float* sb = tile;                  // [TT][padded]
  float* sc = sb + TT * padded;      // [TT][padded]
  float* sx = sc + TT * padded;      // [TT][cols]
  float* sdt = sx + TT * cols;       // [TT] step size
  float* sdecay = sdt + TT;          // [TT]
  const float rate = expf(a.a_log[h]), dt_bias = a.dt_bias[h], d_skip = a.d_skip[h];

  float S[R];
  float* sp = a.state + (((size_t)slot * a.n_heads + h) * vdim + j) * n_state;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int row = part * R + i;
    S[i] = (live && row < n_state) ? sp[row] : 0.f;
  }
  for (int t0 = begin; t0 < end; t0 += TT) {
    const int nt = min(TT, end - t0);
    __syncthreads();
    for (int e = threadIdx.x; e < nt * padded; e += blockDim.x) {
      const int tt = e / padded, d = e - tt * padded;
      const size_t t = (size_t)(t0 + tt);
      sb[e] = d < n_state ? a.b[t * a.bc_stride + g * n_state + d] : 0.f;
      sc[e] = d < n_state ? a.c[t * a.bc_stride + g * n_state + d] : 0.f;
    }
    for (int e = threadIdx.x; e < nt * cols; e += blockDim.x) {
      const int tt = e / cols, cc = e - tt * cols;
      sx[e] = col0 + cc < vdim ? a.x[(size_t)(t0 + tt) * a.x_stride + h * vdim + col0 + cc] : 0.f;
    }
    for (int tt = threadIdx.x; tt < nt; tt += blockDim.x) {
      const float z = a.dt[(size_t)(t0 + tt) * a.dt_stride + h] + dt_bias;
      const float dt = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
      sdt[tt] = dt;
      sdecay[tt] = expf(-rate * dt);
    }
    __syncthreads();
#pragma unroll 4
    for (int tt = 0; tt < nt; ++tt) {
      const float xv = sx[tt * cols + jl];
      const float decay = sdecay[tt], u = sdt[tt] * xv;
      float bt[R], ct[R];
      if (R % 4 == 0) {  // a lane's rows of b and c as whole 16 bytes
#pragma unroll
        for (int i = 0; i < R; i += 4) {
          const float4 b4 = *reinterpret_cast<const float4*>(sb + tt * padded + part * R + i);
          const float4 c4 = *reinterpret_cast<const float4*>(sc + tt * padded + part * R + i);
          bt[i] = b4.x; bt[i + 1] = b4.y; bt[i + 2] = b4.z; bt[i + 3] = b4.w;
          ct[i] = c4.x; ct[i + 1] = c4.y; ct[i + 2] = c4.z; ct[i + 3] = c4.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < R; ++i) {
          bt[i] = sb[tt * padded + part * R + i];
          ct[i] = sc[tt * padded + part * R + i];
        }
      }
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        S[i] = fmaf(decay, S[i], u * bt[i]);
        if (i & 1) y1 = fmaf(S[i], ct[i], y1);
        else y0 = fmaf(S[i], ct[i], y0);
      }
      float y = y0 + y1;
      for (int o = parts >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (part == 0 && live) a.out[(size_t)(t0 + tt) * a.n_heads * vdim + h * vdim + j] = fmaf(d_skip, xv, y);
    }
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int row = part * R + i;
    if (live && row < n_state) sp[row] = S[i];
  }
}

// v = y * silu(z); each of `groups` stretches of the row by its own root mean square; times w.  One block a
// (token, group).
template <typename TO>
__global__ void gated_group_norm_kernel(TO* __restrict__ out, const float* __restrict__ y, const float* __restrict__ z,
                                        int z_stride, const float* __restrict__ w, int width, int groups, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, g = blockIdx.y;
  const int per = width / groups;
  const float* yr = y + (size_t)t * width + g * per;
  const float* zr = z + (size_t)t * z_stride + g * per;
  float acc = 0.f;
  for (int c = threadIdx.x; c < per; c += blockDim.x) {
    const float zv = zr[c];
    const float v = yr[c] * (zv / (1.0f + expf(-zv)));
    acc = fmaf(v, v, acc);
  }
  const float inv = 1.0f / sqrtf(block_sum(acc, scratch) / (float)per + eps);
  for (int c = threadIdx.x; c < per; c += blockDim.x) {
    const float zv = zr[c];
    const float v = yr[c] * (zv / (1.0f + expf(-zv)));
    out[(size_t)t * width + g * per + c] = from_float<TO>((v * inv) * w[g * per + c]);
  }
}

}  // namespace xrt

// out [T, heads * vdim] float32.  x: rows holding heads * vdim floats; b, c: rows holding groups * n_state floats (one
// stride for both); dt: rows holding one raw step size a head.  state: [slots, heads, vdim, n_state].
XRT_EXPORT int xrt_ssd_scan(float* out, const float* x, int x_stride, const float* b, const float* c, int bc_stride,
                            const float* dt, int dt_stride, const float* dt_bias, const float* a_log, const float* d_skip,
                            float* state, const int* cu_seqlens, const int* seq_slot, int n_seqs, int n_heads,
                            int n_groups, int n_state, int vdim, int max_new, cudaStream_t stream) {
  if (n_seqs < 0 || n_heads <= 0 || n_groups <= 0 || n_heads % n_groups || n_state <= 0 || vdim <= 0) return XRT_ERR_ARGUMENT;
  if (n_state > 512 || n_seqs > 65535 || n_heads > 65535) return XRT_ERR_UNSUPPORTED;
  if (n_seqs == 0) return XRT_OK;
  if (max_new < 1) max_new = 1 << 30;
  int r = 1;
  while (r < 16 && (n_state + r - 1) / r > 16) r *= 2;  // rows a lane: 16 lanes a column where the state allows
  int parts = 1;
  while (parts * r < n_state) parts *= 2;
  if (parts > 32) return XRT_ERR_UNSUPPORTED;
  xrt::SsdArgs a;
  a.out = out; a.x = x; a.b = b; a.c = c; a.dt = dt;
  a.x_stride = x_stride; a.bc_stride = bc_stride; a.dt_stride = dt_stride;
  a.dt_bias = dt_bias; a.a_log = a_log; a.d_skip = d_skip;
  a.state = state; a.cu_seqlens = cu_seqlens; a.seq_slot = seq_slot;
  a.n_heads = n_heads; a.heads_per_group = n_heads / n_groups; a.n_state = n_state; a.vdim = vdim;
  a.parts = parts;
  int threads = 128;
  while (threads > 32 && threads / parts >= 2 * vdim) threads /= 2;  // no more lanes than the columns need
  a.cols = threads / parts;
  a.tile_tokens = max_new < 32 ? max_new : 32;
  while (a.tile_tokens > 1 && (size_t)a.tile_tokens * (2 * parts * r + a.cols + 2) * sizeof(float) > 40 * 1024)
    a.tile_tokens /= 2;
  const size_t smem = ((size_t)a.tile_tokens * (2 * parts * r + a.cols + 2)) * sizeof(float);
  dim3 grid(n_seqs, n_heads, (vdim + a.cols - 1) / a.cols);
#define XRT_SSD(R) xrt::launch_kernel(xrt::ssd_scan_kernel<R>, grid, dim3(threads), smem, stream, a)
  if (r == 1) XRT_SSD(1);
  else if (r == 2) XRT_SSD(2);
  else if (r == 4) XRT_SSD(4);
  else if (r == 8) XRT_SSD(8);
  else XRT_SSD(16);
#undef XRT_SSD
  return xrt::launch_status();
}

XRT_EXPORT int xrt_gated_group_norm(void* out, const float* y, const float* z, int z_stride, const float* weight,
                                    int n_tokens, int width, int groups, float eps, int out_dtype, cudaStream_t stream) {
  if (n_tokens < 0 || width <= 0 || groups <= 0 || width % groups || z_stride < width) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  if (groups > 65535) return XRT_ERR_UNSUPPORTED;
  const int per = width / groups;
  const int threads = per >= 1024 ? 256 : (per >= 256 ? 128 : 64);
  XRT_DISPATCH_DTYPE(out_dtype, TO, {
    xrt::launch_kernel(xrt::gated_group_norm_kernel<TO>, dim3(n_tokens, groups), dim3(threads), 0, stream, (TO*)out, y, z,
                       z_stride, weight, width, groups, eps);
  });
  return xrt::launch_status();
}
