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
// `parts` neighbouring lanes, R rows each (which rows: `row_of` in the kernel; rows beyond n_state stay zero);
// the read-out's sum over rows is finished by a butterfly among those lanes, so its order is fixed.  Tiles of
// `tile_tokens` tokens' b, c, x and raw step sizes are brought into shared memory by cp.async, two tiles in flight:
// the next tile lands while this one is worked on.
template <int BYTES>
__device__ __forceinline__ void ssd_cp_async(float* smem, const float* global) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  if (BYTES == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(global) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(global) : "memory");
}

// VEC: 16-byte copies (n_state, cols, vdim and every row stride are multiples of 4 floats, every base 16-byte aligned).
template <int R, bool VEC>
__global__ void __launch_bounds__(128) ssd_scan_kernel(const SsdArgs a) {
  extern __shared__ __align__(16) float tile[];
  pdl_trigger();
  const int parts = a.parts, cols = a.cols, TT = a.tile_tokens, n_state = a.n_state, vdim = a.vdim;
  const int padded = parts * R;
  // a stage: b | c, each [TT][padded]; x [TT][cols]; raw step sizes [TT] (padded to 4); then step size and decay [TT] each
  const int stage_floats = 2 * TT * padded + TT * cols + ((TT + 3) & ~3);
  float* sdt = tile + 2 * stage_floats;
  float* sdecay = sdt + TT;
  if (padded != n_state || vdim % cols != 0)  // rows and columns beyond the head's stay zero
    for (int e = threadIdx.x; e < 2 * stage_floats; e += blockDim.x) tile[e] = 0.f;
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y;
  const int slot = a.seq_slot[s];
  const int begin = a.cu_seqlens[s], end = a.cu_seqlens[s + 1];
  if (slot < 0 || end <= begin) return;
  __syncthreads();
  const int part = threadIdx.x % parts, jl = threadIdx.x / parts;
  const int col0 = blockIdx.z * cols, j = col0 + jl;
  const int g = h / a.heads_per_group;
  const bool live = j < vdim;
  const float rate = expf(a.a_log[h]), dt_bias = a.dt_bias[h], d_skip = a.d_skip[h];
  constexpr int B = VEC ? 16 : 4, E = VEC ? 4 : 1;
  // the lane's i-th row: with four rows or more a lane, every parts-th group of four (the lanes of a column then read
  // neighbouring 16 bytes of b, c and the state: whole lines, all banks), else R neighbouring rows
  auto row_of = [&](int i) { return R % 4 == 0 ? 4 * ((i >> 2) * parts + part) + (i & 3) : part * R + i; };

  auto issue = [&](int t0, int stage) {
    float* sb = tile + stage * stage_floats;
    float* sc = sb + TT * padded;
    float* sx = sc + TT * padded;
    float* sraw = sx + TT * cols;
    const int nt = min(TT, end - t0);
    const int per = n_state / E;
    if (blockDim.x % per == 0) {  // a thread keeps its piece of the row and steps down the tokens: no division a copy
      const int d = (threadIdx.x % per) * E;
      for (int tt = threadIdx.x / per; tt < nt; tt += blockDim.x / per) {
        const size_t at = (size_t)(t0 + tt) * a.bc_stride + g * n_state + d;
        ssd_cp_async<B>(sb + tt * padded + d, a.b + at);
        ssd_cp_async<B>(sc + tt * padded + d, a.c + at);
      }
    } else {
      for (int e = threadIdx.x; e < nt * per; e += blockDim.x) {
        const int tt = e / per, d = (e - tt * per) * E;
        const size_t at = (size_t)(t0 + tt) * a.bc_stride + g * n_state + d;
        ssd_cp_async<B>(sb + tt * padded + d, a.b + at);
        ssd_cp_async<B>(sc + tt * padded + d, a.c + at);
      }
    }
    const int xper = cols / E;
    for (int e = threadIdx.x; e < nt * xper; e += blockDim.x) {
      const int tt = e / xper, cc = (e - tt * xper) * E;
      if (col0 + cc < vdim) ssd_cp_async<B>(sx + tt * cols + cc, a.x + (size_t)(t0 + tt) * a.x_stride + h * vdim + col0 + cc);
    }
    for (int tt = threadIdx.x; tt < nt; tt += blockDim.x)
      ssd_cp_async<4>(sraw + tt, a.dt + (size_t)(t0 + tt) * a.dt_stride + h);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float S[R];
  float* sp = a.state + (((size_t)slot * a.n_heads + h) * vdim + j) * n_state;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int row = row_of(i);
    S[i] = (live && row < n_state) ? sp[row] : 0.f;
  }
  issue(begin, 0);
  int stage = 0;
  for (int t0 = begin; t0 < end; t0 += TT, stage ^= 1) {
    const int nt = min(TT, end - t0);
    if (t0 + TT < end) {
      issue(t0 + TT, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* sb = tile + stage * stage_floats;
    const float* sc = sb + TT * padded;
    const float* sx = sc + TT * padded;
    const float* sraw = sx + TT * cols;
    for (int tt = threadIdx.x; tt < nt; tt += blockDim.x) {
      const float z = sraw[tt] + dt_bias;
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
          const float4 b4 = *reinterpret_cast<const float4*>(sb + tt * padded + row_of(i));
          const float4 c4 = *reinterpret_cast<const float4*>(sc + tt * padded + row_of(i));
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
    __syncthreads();  // the stage is written again by the copies of the tile after the next
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int row = row_of(i);
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
  a.tile_tokens = max_new < 16 ? max_new : 16;
  auto floats = [&](int tt) { return (size_t)2 * (2 * tt * parts * r + tt * a.cols + ((tt + 3) & ~3)) + 2 * tt; };
  while (a.tile_tokens > 1 && floats(a.tile_tokens) * sizeof(float) > 44 * 1024) a.tile_tokens /= 2;
  const size_t smem = floats(a.tile_tokens) * sizeof(float);
  const bool vec = n_state % 4 == 0 && a.cols % 4 == 0 && vdim % 4 == 0 && x_stride % 4 == 0 && bc_stride % 4 == 0 &&
                   (((uintptr_t)x | (uintptr_t)b | (uintptr_t)c) & 15) == 0;
  dim3 grid(n_seqs, n_heads, (vdim + a.cols - 1) / a.cols);
#define XRT_SSD(R)                                                                                              \
  do {                                                                                                          \
    if (vec) xrt::launch_kernel(xrt::ssd_scan_kernel<R, true>, grid, dim3(threads), smem, stream, a);          \
    else xrt::launch_kernel(xrt::ssd_scan_kernel<R, false>, grid, dim3(threads), smem, stream, a);             \
  } while (0)
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
