// Bandwidth-bound kernels of the Llama / GPT-2 trainers (sm_100a): RMSNorm, LayerNorm, RoPE,
// SwiGLU, bias + GELU, fused softmax cross-entropy, embedding, and a flat fused AdamW.  Every one
// makes a single pass over its operands with 16-byte accesses and keeps row statistics
// in registers / shared memory; the torch-eager equivalents (several kernels and
// temporaries each) are the baseline they replace.  The reference trainer gets these
// ops from torch (benchmarks/train_llama7b_dp_pp_lowbit.py:158-165,248).
//
// C linkage, raw pointers + stream, async, cudaError_t returned as int.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ew {

typedef __nv_bfloat16 bf16;

struct alignas(16) Bf8 {
  bf16 v[8];
};

__device__ __forceinline__ void load8(const bf16* p, float (&f)[8]) {
  const Bf8 raw = *reinterpret_cast<const Bf8*>(p);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(raw.v[i]);
}
__device__ __forceinline__ void store8(bf16* p, const float (&f)[8]) {
  Bf8 raw;
#pragma unroll
  for (int i = 0; i < 8; ++i) raw.v[i] = __float2bfloat16_rn(f[i]);
  *reinterpret_cast<Bf8*>(p) = raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// block-wide sum for up to 1024 threads; every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* scratch /*[33]*/) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x + 31) / 32 ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x + 31) / 32 ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// ---------------------------------------------------------------------------
// RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w        (H % 8 == 0)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                   float* __restrict__ rstd_out, int rows, int H, float eps) {
  __shared__ float scratch[33];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const bf16* xr = x + (size_t)row * H;
    float ss = 0.0f;
    for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
      float f[8];
      load8(xr + c, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (threadIdx.x == 0) rstd_out[row] = rstd;
    bf16* yr = y + (size_t)row * H;
    for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
      float f[8], g[8];
      load8(xr + c, f);
      load8(w + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * g[i];
      store8(yr + c, f);
    }
  }
}

// dx = rstd * (dy*w - x * rstd^2 * mean(dy*w*x)) [+ dres];  dw += sum_rows dy * x * rstd (fp32)
// Each CTA walks rows blockIdx.x, +gridDim.x, ... and keeps its dw partial in registers
// (thread t owns columns t*8 + k*blockDim*8).  A row is read once: x and dy stay in registers
// (as packed bf16) across the reduction, the next row's loads are issued before the reduction
// of the current one, and the reduction costs one barrier (warp partials in a double-buffered
// scratch, every thread adds them up itself).  At the end a CTA writes its dw partial to its
// row of `partials` ([gridDim.x][H] fp32) and colsum_add_kernel folds the rows into dw: H
// atomic adds per CTA on the same H addresses used to cost a third of the kernel's time.
// `dres` (HAS_RES): the gradient that reaches the same input through the residual connection,
// added to dx here instead of by a separate add kernel.
template <int MAX_ITERS, bool HAS_RES>
__global__ void __launch_bounds__(512)
rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                   const bf16* __restrict__ w, const float* __restrict__ rstd,
                   const bf16* __restrict__ dres, bf16* __restrict__ dx,
                   float* __restrict__ partials, int rows, int H) {
  __shared__ float partial[2][16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  float acc[MAX_ITERS][8], fw[MAX_ITERS][8];
  Bf8 cx[MAX_ITERS], cg[MAX_ITERS], nx[MAX_ITERS], ng[MAX_ITERS];
#pragma unroll
  for (int k = 0; k < MAX_ITERS; ++k) {
    const int c = (threadIdx.x + k * blockDim.x) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[k][i] = fw[k][i] = 0.0f;
    if (c < H) load8(w + c, fw[k]);
  }
  auto fetch = [&](int row, Bf8 (&bx)[MAX_ITERS], Bf8 (&bg)[MAX_ITERS]) {
#pragma unroll
    for (int k = 0; k < MAX_ITERS; ++k) {
      const int c = (threadIdx.x + k * blockDim.x) * 8;
      if (c < H) {
        bx[k] = *reinterpret_cast<const Bf8*>(x + (size_t)row * H + c);
        bg[k] = *reinterpret_cast<const Bf8*>(dy + (size_t)row * H + c);
      }
    }
  };
  int row = blockIdx.x;
  if (row < rows) fetch(row, cx, cg);
  int parity = 0;
  for (; row < rows; row += gridDim.x, parity ^= 1) {
    const int next = row + gridDim.x;
    if (next < rows) fetch(next, nx, ng);
    const float rs = rstd[row];
    float dot = 0.0f;
#pragma unroll
    for (int k = 0; k < MAX_ITERS; ++k) {
      const int c = (threadIdx.x + k * blockDim.x) * 8;
      if (c < H) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float fx = __bfloat162float(cx[k].v[i]), fg = __bfloat162float(cg[k].v[i]);
          dot += fg * fw[k][i] * fx;
          acc[k][i] += fg * fx * rs;
        }
      }
    }
    dot = warp_sum(dot);
    if (lane == 0) partial[parity][warp] = dot;
    __syncthreads();  // the other buffer is free again: its readers passed the previous barrier
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) total += i < nwarps ? partial[parity][i] : 0.0f;
    const float coef = total * rs * rs * rs / (float)H;
    bf16* dr = dx + (size_t)row * H;
#pragma unroll
    for (int k = 0; k < MAX_ITERS; ++k) {
      const int c = (threadIdx.x + k * blockDim.x) * 8;
      if (c < H) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float fx = __bfloat162float(cx[k].v[i]), fg = __bfloat162float(cg[k].v[i]);
          o[i] = fg * fw[k][i] * rs - fx * coef;
        }
        if constexpr (HAS_RES) {
          float rr[8];
          load8(dres + (size_t)row * H + c, rr);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += rr[i];
        }
        store8(dr + c, o);
        cx[k] = nx[k];
        cg[k] = ng[k];
      }
    }
  }
#pragma unroll
  for (int k = 0; k < MAX_ITERS; ++k) {
    const int c = (threadIdx.x + k * blockDim.x) * 8;
    if (c < H) {
      float* dst = partials + (size_t)blockIdx.x * H + c;
      *reinterpret_cast<float4*>(dst) = make_float4(acc[k][0], acc[k][1], acc[k][2], acc[k][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[k][4], acc[k][5], acc[k][6], acc[k][7]);
    }
  }
}

// out[c] += sum over p < nparts of partials[p * width + c] for the `width` columns of a
// partial row; columns [0, split) belong to out_a, columns [split, width) to out_b (at
// out_b[c - split]).  blockDim = (32, 32): a CTA owns 32 columns, its 32 thread rows split
// the partial rows (a few loads each, all in flight at once), shared memory folds them.
__global__ void __launch_bounds__(1024)
colsum_add_kernel(const float* __restrict__ partials, float* __restrict__ out_a,
                  float* __restrict__ out_b, int nparts, int width, int split) {
  __shared__ float fold[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.0f;
  if (c < width) {
    int p = threadIdx.y;
    for (; p + 96 < nparts; p += 128) {
      const float a0 = partials[(size_t)p * width + c];
      const float a1 = partials[(size_t)(p + 32) * width + c];
      const float a2 = partials[(size_t)(p + 64) * width + c];
      const float a3 = partials[(size_t)(p + 96) * width + c];
      s += (a0 + a1) + (a2 + a3);
    }
    for (; p < nparts; p += 32) s += partials[(size_t)p * width + c];
  }
  fold[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < width) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) t += fold[i][threadIdx.x];
    if (c < split) out_a[c] += t;
    else out_b[c - split] += t;
  }
}

// ---------------------------------------------------------------------------
// LayerNorm (GPT-2): y = (x - mean) * rstd * w + b.  One warp per row, the row held in
// registers between the statistics and the output (one read of x).  H <= 32 * 8 * MAX_ITERS
// (the launchers instantiate 2 and 4: H up to 1024).
// ---------------------------------------------------------------------------
template <int MAX_ITERS>
__global__ void __launch_bounds__(256)
layernorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                     const bf16* __restrict__ b, bf16* __restrict__ y,
                     float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int H,
                     float eps) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  for (int row = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); row < rows;
       row += gridDim.x * warps_per_cta) {
    const bf16* xr = x + (size_t)row * H;
    float f[MAX_ITERS][8];
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < MAX_ITERS; ++k) {
      const int c = (lane + k * 32) * 8;
      if (c < H) {
        load8(xr + c, f[k]);
#pragma unroll
        for (int i = 0; i < 8; ++i) sum += f[k][i];
      }
    }
    const float mean = warp_sum(sum) / (float)H;
    float var = 0.0f;
#pragma unroll
    for (int k = 0; k < MAX_ITERS; ++k) {
      const int c = (lane + k * 32) * 8;
      if (c < H) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float d = f[k][i] - mean;
          var += d * d;
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(var) / (float)H + eps);
    if (lane == 0) {
      mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
    bf16* yr = y + (size_t)row * H;
#pragma unroll
    for (int k = 0; k < MAX_ITERS; ++k) {
      const int c = (lane + k * 32) * 8;
      if (c < H) {
        float g[8], bb[8], o[8];
        load8(w + c, g);
        load8(b + c, bb);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (f[k][i] - mean) * rstd * g[i] + bb[i];
        store8(yr + c, o);
      }
    }
  }
}

// LayerNorm backward, one row per CTA pass (H <= 1024: at most 128 threads, thread t owns
// columns [8t, 8t + 8)).  Same shape as rmsnorm_bwd_kernel: the next row's x and dy are
// requested before the current row's reduction, the two row sums cost one barrier (warp
// partials in a double-buffered scratch), dw / db partials stay in registers and leave as one
// [dw | db] row of `partials` per CTA.  Against the one-warp-per-row kernel it keeps 16 x
// fewer values per thread (40 instead of 160 registers of row state), so sixteen CTAs fit an
// SM and a row's latency chain is an eighth as long.
__global__ void __launch_bounds__(128)
layernorm_bwd_row_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                         const bf16* __restrict__ w, const float* __restrict__ mean,
                         const float* __restrict__ rstd, bf16* __restrict__ dx,
                         float* __restrict__ partials, int rows, int H) {
  __shared__ float partial[2][2][4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  const int c = threadIdx.x * 8;
  const bool live = c < H;
  float aw[8], ab[8], fw[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) aw[i] = ab[i] = fw[i] = 0.0f;
  if (live) load8(w + c, fw);
  Bf8 cx, cg, nx, ng;
  auto fetch = [&](int row, Bf8& bx, Bf8& bg) {
    if (live) {
      bx = *reinterpret_cast<const Bf8*>(x + (size_t)row * H + c);
      bg = *reinterpret_cast<const Bf8*>(dy + (size_t)row * H + c);
    }
  };
  int row = blockIdx.x;
  if (row < rows) fetch(row, cx, cg);
  int parity = 0;
  const float inv_h = 1.0f / (float)H;
  for (; row < rows; row += gridDim.x, parity ^= 1) {
    const int next = row + gridDim.x;
    if (next < rows) fetch(next, nx, ng);
    const float mu = mean[row], rs = rstd[row];
    float xh[8], g[8];
    float s1 = 0.0f, s2 = 0.0f;
    if (live) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float fx = __bfloat162float(cx.v[i]), fg = __bfloat162float(cg.v[i]);
        xh[i] = (fx - mu) * rs;
        g[i] = fg * fw[i];
        s1 += g[i];
        s2 += g[i] * xh[i];
        aw[i] += fg * xh[i];
        ab[i] += fg;
      }
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if (lane == 0) {
      partial[parity][0][warp] = s1;
      partial[parity][1][warp] = s2;
    }
    __syncthreads();  // the other buffer is free again: its readers passed the previous barrier
    float t1 = 0.0f, t2 = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      t1 += i < nwarps ? partial[parity][0][i] : 0.0f;
      t2 += i < nwarps ? partial[parity][1][i] : 0.0f;
    }
    t1 *= inv_h;
    t2 *= inv_h;
    if (live) {
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = rs * (g[i] - t1 - xh[i] * t2);
      store8(dx + (size_t)row * H + c, o);
      cx = nx;
      cg = ng;
    }
  }
  if (live) {
    float* dst = partials + (size_t)blockIdx.x * 2 * H + c;
    *reinterpret_cast<float4*>(dst) = make_float4(aw[0], aw[1], aw[2], aw[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(aw[4], aw[5], aw[6], aw[7]);
    *reinterpret_cast<float4*>(dst + H) = make_float4(ab[0], ab[1], ab[2], ab[3]);
    *reinterpret_cast<float4*>(dst + H + 4) = make_float4(ab[4], ab[5], ab[6], ab[7]);
  }
}

// ---------------------------------------------------------------------------
// bias + GELU (tanh form) on a [rows, C] GEMM output: y = gelu(x + bias).
// Backward recomputes from x and bias: dx = dy * gelu'(x + bias), dbias += colsum(dx).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float tanh_fast(float v) {
  float r;
  asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
constexpr float kGeluK = 0.7978845608028654f;  // sqrt(2 / pi)
constexpr float kGeluC = 0.044715f;

__global__ void __launch_bounds__(256)
bias_gelu_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ bias,
                     bf16* __restrict__ y, long long rows, int C) {
  const int vec = C / 8;
  const long long total = rows * vec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % vec) * 8;
    float u[8], bb[8];
    load8(x + i * 8, u);
    load8(bias + c, bb);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float v = u[k] + bb[k];
      u[k] = 0.5f * v * (1.0f + tanh_fast(kGeluK * (v + kGeluC * v * v * v)));
    }
    store8(y + i * 8, u);
  }
}

// grid: (C / (8 * blockDim.x) column tiles, row strips).  Thread t of a column tile owns 8
// columns and walks its strip's rows, so the bias gradient needs 8 atomics per thread.
__global__ void __launch_bounds__(256)
bias_gelu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                     const bf16* __restrict__ bias, bf16* __restrict__ dx,
                     float* __restrict__ dbias, long long rows, int C) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  float bb[8], acc[8];
  load8(bias + c, bb);
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
  // four rows of loads in flight per thread (one row at a time left the kernel at a third of
  // the copy rate)
  for (long long r0 = blockIdx.y; r0 < rows; r0 += 4LL * gridDim.y) {
    Bf8 bu[4], bd[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long r = r0 + (long long)j * gridDim.y;
      if (r < rows) {
        bu[j] = *reinterpret_cast<const Bf8*>(x + r * C + c);
        bd[j] = *reinterpret_cast<const Bf8*>(dy + r * C + c);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long r = r0 + (long long)j * gridDim.y;
      if (r >= rows) continue;
      float d[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float v = __bfloat162float(bu[j].v[k]) + bb[k];
        const float t = tanh_fast(kGeluK * (v + kGeluC * v * v * v));
        const float dg = 0.5f * (1.0f + t) +
                         0.5f * v * (1.0f - t * t) * kGeluK * (1.0f + 3.0f * kGeluC * v * v);
        d[k] = __bfloat162float(bd[j].v[k]) * dg;
        acc[k] += d[k];
      }
      store8(dx + r * C + c, d);
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) atomicAdd(dbias + c + k, acc[k]);
}

// ---------------------------------------------------------------------------
// RoPE (rotate-half convention), in place on a [tokens, heads, head_dim] slice of a
// wider row: element (t, h, d) sits at x[t * row_stride + h * head_dim + d].
// cos/sin: [seq, head_dim/2] fp32; position of token t is t % seq.
// sign = +1 forward, -1 backward (the transposed rotation).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rope_kernel(bf16* __restrict__ x, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
            long long tokens, int heads, int head_dim, long long row_stride, int seq, float sign) {
  const int half = head_dim / 2;
  const int vec_per_head = half / 8;
  const long long total = tokens * heads * vec_per_head;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_head);
    const long long th = i / vec_per_head;
    const int h = (int)(th % heads);
    const long long t = th / heads;
    const int pos = (int)(t % seq);
    bf16* base = x + t * row_stride + (long long)h * head_dim + v * 8;
    float a[8], b[8];
    load8(base, a);
    load8(base + half, b);
    const float* c = cos_t + (size_t)pos * half + v * 8;
    const float* s = sin_t + (size_t)pos * half + v * 8;
    float ra[8], rb[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float cs = c[k], sn = s[k] * sign;
      ra[k] = a[k] * cs - b[k] * sn;
      rb[k] = b[k] * cs + a[k] * sn;
    }
    store8(base, ra);
    store8(base + half, rb);
  }
}

// ---------------------------------------------------------------------------
// SwiGLU on a fused [tokens, 2F] projection (gate | up): h = silu(gate) * up
// ---------------------------------------------------------------------------
// Two independent 8-element groups per thread and iteration: all loads of both are issued
// before the first result is needed (one group per iteration left the kernels at half the copy
// rate: too few bytes in flight per thread for five streams).
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ h, long long tokens, int F) {
  const int vec = F / 8;
  const long long total = tokens * vec;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < total;
       i0 += 2 * stride) {
    const long long i1 = i0 + stride;
    const bool two = i1 < total;
    const long long t0 = i0 / vec, t1 = two ? i1 / vec : t0;
    const int c0 = (int)(i0 - t0 * vec) * 8, c1 = two ? (int)(i1 - t1 * vec) * 8 : c0;
    Bf8 g0 = *reinterpret_cast<const Bf8*>(gu + t0 * 2 * F + c0);
    Bf8 u0 = *reinterpret_cast<const Bf8*>(gu + t0 * 2 * F + F + c0);
    Bf8 g1 = *reinterpret_cast<const Bf8*>(gu + t1 * 2 * F + c1);
    Bf8 u1 = *reinterpret_cast<const Bf8*>(gu + t1 * 2 * F + F + c1);
    float o[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float g = __bfloat162float(g0.v[k]);
      o[k] = g / (1.0f + __expf(-g)) * __bfloat162float(u0.v[k]);
    }
    store8(h + t0 * F + c0, o);
    if (two) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float g = __bfloat162float(g1.v[k]);
        o[k] = g / (1.0f + __expf(-g)) * __bfloat162float(u1.v[k]);
      }
      store8(h + t1 * F + c1, o);
    }
  }
}

__device__ __forceinline__ void swiglu_bwd8(const Bf8& g, const Bf8& u, const Bf8& d,
                                            float (&dg)[8], float (&du)[8]) {
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float gk = __bfloat162float(g.v[k]), uk = __bfloat162float(u.v[k]);
    const float dk = __bfloat162float(d.v[k]);
    const float sg = 1.0f / (1.0f + __expf(-gk));
    const float silu = gk * sg;
    dg[k] = dk * uk * (sg + silu * (1.0f - sg));
    du[k] = dk * silu;
  }
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const bf16* __restrict__ gu, const bf16* __restrict__ dh,
                  bf16* __restrict__ dgu, long long tokens, int F) {
  const int vec = F / 8;
  const long long total = tokens * vec;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < total;
       i0 += 2 * stride) {
    const long long i1 = i0 + stride;
    const bool two = i1 < total;
    const long long t0 = i0 / vec, t1 = two ? i1 / vec : t0;
    const int c0 = (int)(i0 - t0 * vec) * 8, c1 = two ? (int)(i1 - t1 * vec) * 8 : c0;
    const Bf8 g0 = *reinterpret_cast<const Bf8*>(gu + t0 * 2 * F + c0);
    const Bf8 u0 = *reinterpret_cast<const Bf8*>(gu + t0 * 2 * F + F + c0);
    const Bf8 d0 = *reinterpret_cast<const Bf8*>(dh + t0 * F + c0);
    const Bf8 g1 = *reinterpret_cast<const Bf8*>(gu + t1 * 2 * F + c1);
    const Bf8 u1 = *reinterpret_cast<const Bf8*>(gu + t1 * 2 * F + F + c1);
    const Bf8 d1 = *reinterpret_cast<const Bf8*>(dh + t1 * F + c1);
    float dg[8], du[8];
    swiglu_bwd8(g0, u0, d0, dg, du);
    store8(dgu + t0 * 2 * F + c0, dg);
    store8(dgu + t0 * 2 * F + F + c0, du);
    if (two) {
      swiglu_bwd8(g1, u1, d1, dg, du);
      store8(dgu + t1 * 2 * F + c1, dg);
      store8(dgu + t1 * 2 * F + F + c1, du);
    }
  }
}

// ---------------------------------------------------------------------------
// Fused softmax cross-entropy: one CTA per row of logits [rows, V] (V % 8 == 0).
// loss_out[row] = logsumexp - logit[target] (0 for ignored rows); the logits are
// overwritten in place by dlogits = (softmax - onehot) * grad_scale[0].
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(512)
cross_entropy_kernel(bf16* __restrict__ logits, const long long* __restrict__ targets,
                     float* __restrict__ loss_out, const float* __restrict__ grad_scale,
                     int rows, int V, long long ignore_index) {
  __shared__ float scratch[33];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    bf16* lr = logits + (size_t)row * V;
    const long long tgt = targets[row];
    float m = -INFINITY;
    for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
      float f[8];
      load8(lr + c, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) m = fmaxf(m, f[i]);
    }
    m = block_max(m, scratch);
    float s = 0.0f;
    for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
      float f[8];
      load8(lr + c, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += __expf(f[i] - m);
    }
    s = block_sum(s, scratch);
    const bool ignored = tgt == ignore_index || tgt < 0 || tgt >= V;
    const float lse = m + logf(s);
    if (threadIdx.x == 0)
      loss_out[row] = ignored ? 0.0f : lse - __bfloat162float(lr[tgt]);
    __syncthreads();  // the target logit is read before anybody overwrites it
    const float scale = ignored ? 0.0f : grad_scale[0];
    const float inv = 1.0f / s;
    for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
      float f[8];
      load8(lr + c, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float p = __expf(f[i] - m) * inv;
        if (c + i == tgt) p -= 1.0f;
        f[i] = p * scale;
      }
      store8(lr + c, f);
    }
  }
}

// ---------------------------------------------------------------------------
// Embedding lookup and its gradient (fp32 accumulation with atomics)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ table,
                     bf16* __restrict__ out, long long tokens, int H, int vocab) {
  const int vec = H / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < tokens * vec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec;
    const int c = (int)(i - t * vec) * 8;
    long long id = ids[t];
    if (id < 0 || id >= vocab) id = 0;
    *reinterpret_cast<Bf8*>(out + t * H + c) =
        *reinterpret_cast<const Bf8*>(table + id * H + c);
  }
}

__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ dout,
                     float* __restrict__ dtable, long long tokens, int H, int vocab) {
  const int vec = H / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < tokens * vec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec;
    const int c = (int)(i - t * vec) * 8;
    const long long id = ids[t];
    if (id < 0 || id >= vocab) continue;
    float f[8];
    load8(dout + t * H + c, f);
#pragma unroll
    for (int k = 0; k < 8; ++k) atomicAdd(dtable + id * H + c + k, f[k]);
  }
}

// ---------------------------------------------------------------------------
// Flat fused AdamW over fp32 master weights; also refreshes the bf16 working copy and
// (optionally) zeroes the gradient for the next step.  n % 4 == 0 buffers, 16-B aligned.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ master, bf16* __restrict__ param_bf16, float* __restrict__ grad,
             float* __restrict__ exp_avg, float* __restrict__ exp_avg_sq, long long n, float lr,
             float beta1, float beta2, float eps, float weight_decay, float bias1, float bias2,
             float grad_scale, int zero_grad) {
  const long long vecs = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < vecs;
       i += (long long)gridDim.x * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(master)[i];
    float4 g = reinterpret_cast<float4*>(grad)[i];
    float4 m = reinterpret_cast<float4*>(exp_avg)[i];
    float4 v = reinterpret_cast<float4*>(exp_avg_sq)[i];
    float* pp = &p.x; float* gg = &g.x; float* mm = &m.x; float* vv = &v.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = gg[k] * grad_scale;
      mm[k] = beta1 * mm[k] + (1.0f - beta1) * gk;
      vv[k] = beta2 * vv[k] + (1.0f - beta2) * gk * gk;
      const float mhat = mm[k] / bias1;
      const float vhat = vv[k] / bias2;
      pp[k] = pp[k] * (1.0f - lr * weight_decay) - lr * mhat / (sqrtf(vhat) + eps);
    }
    reinterpret_cast<float4*>(master)[i] = p;
    reinterpret_cast<float4*>(exp_avg)[i] = m;
    reinterpret_cast<float4*>(exp_avg_sq)[i] = v;
    if (zero_grad) reinterpret_cast<float4*>(grad)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (param_bf16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(p.z, p.w);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(param_bf16)[i] = packed;
    }
  }
}

// SGD with momentum over flat fp32 buffers (ResNet DDP trainer)
__global__ void __launch_bounds__(256)
sgd_momentum_kernel(float* __restrict__ param, float* __restrict__ grad, float* __restrict__ mom,
                    long long n, float lr, float momentum, float weight_decay, float grad_scale,
                    int zero_grad) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float g = grad[i] * grad_scale + weight_decay * param[i];
    const float b = momentum * mom[i] + g;
    mom[i] = b;
    param[i] -= lr * b;
    if (zero_grad) grad[i] = 0.0f;
  }
}

static int grid_for(long long work, int threads) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long g = (work + threads - 1) / threads;
  const long long cap = (long long)sms * 8;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace ew

using namespace ew;

extern "C" {

int bcom_rmsnorm_fwd(const void* x, const void* w, void* y, void* rstd, int rows, int H,
                     float eps, void* stream) {
  if (rows <= 0) return 0;
  if (H % 8) return (int)cudaErrorInvalidValue;
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  rmsnorm_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)x, (const bf16*)w, (bf16*)y, (float*)rstd, rows, H, eps);
  return (int)cudaGetLastError();
}

// `partials`: fp32 scratch of at least bcom_norm_bwd_scratch_elems(H, layernorm) elements,
// private to the call until it has run.  `dres`: optional bf16 [rows, H] added to dx.
static const int kRmsBwdMaxCtas = 148 * 2;
static const int kLnBwdMaxCtas = 148 * 4;

long long bcom_norm_bwd_scratch_elems(int H, int layernorm) {
  return layernorm ? (long long)kLnBwdMaxCtas * 2 * H : (long long)kRmsBwdMaxCtas * H;
}

int bcom_rmsnorm_bwd(const void* dy, const void* x, const void* w, const void* rstd,
                     const void* dres, void* dx, void* dw_fp32, void* partials, int rows, int H,
                     void* stream) {
  if (rows <= 0) return 0;
  if (H % 8) return (int)cudaErrorInvalidValue;
  const int grid = rows < kRmsBwdMaxCtas ? rows : kRmsBwdMaxCtas;
  const int iters = (H / 8 + 511) / 512;
  cudaStream_t st = (cudaStream_t)stream;
#define BCOM_RMS_BWD(N)                                                                       \
  do {                                                                                        \
    if (dres)                                                                                 \
      rmsnorm_bwd_kernel<N, true><<<grid, 512, 0, st>>>(                                      \
          (const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)rstd,                \
          (const bf16*)dres, (bf16*)dx, (float*)partials, rows, H);                           \
    else                                                                                      \
      rmsnorm_bwd_kernel<N, false><<<grid, 512, 0, st>>>(                                     \
          (const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)rstd, nullptr,       \
          (bf16*)dx, (float*)partials, rows, H);                                              \
  } while (0)
  if (iters <= 1) BCOM_RMS_BWD(1);
  else if (iters <= 2) BCOM_RMS_BWD(2);
  else if (iters <= 4) BCOM_RMS_BWD(4);
  else return (int)cudaErrorInvalidValue;  // H up to 16384
#undef BCOM_RMS_BWD
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return (int)err;
  colsum_add_kernel<<<(H + 31) / 32, dim3(32, 32), 0, st>>>(
      (const float*)partials, (float*)dw_fp32, nullptr, grid, H, H);
  return (int)cudaGetLastError();
}

// LayerNorm over rows of H <= 1024 elements (H % 8 == 0; one warp keeps a row in
// registers); mean / rstd: fp32 [rows].
int bcom_layernorm_fwd(const void* x, const void* w, const void* b, void* y, void* mean,
                       void* rstd, int rows, int H, float eps, void* stream) {
  if (rows <= 0) return 0;
  if (H % 8 || H > 1024) return (int)cudaErrorInvalidValue;
  const int warps = 8;
  const int want = (rows + warps - 1) / warps;
  const int grid = want < 148 * 8 ? want : 148 * 8;
  cudaStream_t st = (cudaStream_t)stream;
  const int iters = (H / 8 + 31) / 32;
#define BCOM_LN_FWD(N)                                                                       \
  layernorm_fwd_kernel<N><<<grid, warps * 32, 0, st>>>(                                       \
      (const bf16*)x, (const bf16*)w, (const bf16*)b, (bf16*)y, (float*)mean, (float*)rstd,  \
      rows, H, eps)
  if (iters <= 2) BCOM_LN_FWD(2);
  else BCOM_LN_FWD(4);
#undef BCOM_LN_FWD
  return (int)cudaGetLastError();
}

// dw / db: fp32 [H], accumulated into (not overwritten); `partials`: see bcom_rmsnorm_bwd.
int bcom_layernorm_bwd(const void* dy, const void* x, const void* w, const void* mean,
                       const void* rstd, void* dx, void* dw_fp32, void* db_fp32, void* partials,
                       int rows, int H, void* stream) {
  if (rows <= 0) return 0;
  if (H % 8 || H > 1024) return (int)cudaErrorInvalidValue;
  const int grid = rows < kLnBwdMaxCtas ? rows : kLnBwdMaxCtas;
  const int threads = ((H / 8 + 31) / 32) * 32;
  cudaStream_t st = (cudaStream_t)stream;
  layernorm_bwd_row_kernel<<<grid, threads, 0, st>>>(
      (const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)mean, (const float*)rstd,
      (bf16*)dx, (float*)partials, rows, H);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return (int)err;
  // a partial row is [dw | db]
  colsum_add_kernel<<<(2 * H + 31) / 32, dim3(32, 32), 0, st>>>(
      (const float*)partials, (float*)dw_fp32, (float*)db_fp32, grid, 2 * H, H);
  return (int)cudaGetLastError();
}

int bcom_bias_gelu_fwd(const void* x, const void* bias, void* y, long long rows, int C,
                       void* stream) {
  if (rows <= 0) return 0;
  if (C % 8) return (int)cudaErrorInvalidValue;
  bias_gelu_fwd_kernel<<<grid_for(rows * (C / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)x, (const bf16*)bias, (bf16*)y, rows, C);
  return (int)cudaGetLastError();
}

// dbias: fp32 [C], accumulated into.
int bcom_bias_gelu_bwd(const void* dy, const void* x, const void* bias, void* dx,
                       void* dbias_fp32, long long rows, int C, void* stream) {
  if (rows <= 0) return 0;
  if (C % 8) return (int)cudaErrorInvalidValue;
  const int threads = 128;
  const int col_tiles = (C / 8 + threads - 1) / threads;
  int strips = (148 * 4 + col_tiles - 1) / col_tiles;
  if (strips > rows) strips = (int)rows;
  if (strips > 65535) strips = 65535;
  bias_gelu_bwd_kernel<<<dim3(col_tiles, strips), threads, 0, (cudaStream_t)stream>>>(
      (const bf16*)dy, (const bf16*)x, (const bf16*)bias, (bf16*)dx, (float*)dbias_fp32, rows, C);
  return (int)cudaGetLastError();
}

int bcom_rope(void* x, const void* cos_t, const void* sin_t, long long tokens, int heads,
              int head_dim, long long row_stride, int seq, int backward, void* stream) {
  if (tokens <= 0) return 0;
  if (head_dim % 16 || row_stride % 8) return (int)cudaErrorInvalidValue;
  const long long total = tokens * heads * (head_dim / 16);
  rope_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
      (bf16*)x, (const float*)cos_t, (const float*)sin_t, tokens, heads, head_dim, row_stride,
      seq, backward ? -1.0f : 1.0f);
  return (int)cudaGetLastError();
}

int bcom_swiglu_fwd(const void* gate_up, void* h, long long tokens, int F, void* stream) {
  if (tokens <= 0) return 0;
  if (F % 8) return (int)cudaErrorInvalidValue;
  swiglu_fwd_kernel<<<grid_for(tokens * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)gate_up, (bf16*)h, tokens, F);
  return (int)cudaGetLastError();
}

int bcom_swiglu_bwd(const void* gate_up, const void* dh, void* dgate_up, long long tokens, int F,
                    void* stream) {
  if (tokens <= 0) return 0;
  if (F % 8) return (int)cudaErrorInvalidValue;
  swiglu_bwd_kernel<<<grid_for(tokens * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)gate_up, (const bf16*)dh, (bf16*)dgate_up, tokens, F);
  return (int)cudaGetLastError();
}

int bcom_cross_entropy(void* logits, const void* targets, void* loss_out, const void* grad_scale,
                       int rows, int V, long long ignore_index, void* stream) {
  if (rows <= 0) return 0;
  if (V % 8) return (int)cudaErrorInvalidValue;
  const int grid = rows < 148 * 4 ? rows : 148 * 4;
  cross_entropy_kernel<<<grid, 512, 0, (cudaStream_t)stream>>>(
      (bf16*)logits, (const long long*)targets, (float*)loss_out, (const float*)grad_scale, rows,
      V, ignore_index);
  return (int)cudaGetLastError();
}

int bcom_embedding_fwd(const void* ids, const void* table, void* out, long long tokens, int H,
                       int vocab, void* stream) {
  if (tokens <= 0) return 0;
  if (H % 8) return (int)cudaErrorInvalidValue;
  embedding_fwd_kernel<<<grid_for(tokens * (H / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const long long*)ids, (const bf16*)table, (bf16*)out, tokens, H, vocab);
  return (int)cudaGetLastError();
}

int bcom_embedding_bwd(const void* ids, const void* dout, void* dtable_fp32, long long tokens,
                       int H, int vocab, void* stream) {
  if (tokens <= 0) return 0;
  if (H % 8) return (int)cudaErrorInvalidValue;
  embedding_bwd_kernel<<<grid_for(tokens * (H / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const long long*)ids, (const bf16*)dout, (float*)dtable_fp32, tokens, H, vocab);
  return (int)cudaGetLastError();
}

int bcom_adamw(void* master, void* param_bf16, void* grad, void* exp_avg, void* exp_avg_sq,
               long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
               int step, float grad_scale, int zero_grad, void* stream) {
  if (n <= 0) return 0;
  if (n % 4) return (int)cudaErrorInvalidValue;
  const float bias1 = 1.0f - powf(beta1, (float)step);
  const float bias2 = 1.0f - powf(beta2, (float)step);
  adamw_kernel<<<grid_for(n / 4, 256), 256, 0, (cudaStream_t)stream>>>(
      (float*)master, (bf16*)param_bf16, (float*)grad, (float*)exp_avg, (float*)exp_avg_sq, n, lr,
      beta1, beta2, eps, weight_decay, bias1, bias2, grad_scale, zero_grad);
  return (int)cudaGetLastError();
}

int bcom_sgd_momentum(void* param, void* grad, void* mom, long long n, float lr, float momentum,
                      float weight_decay, float grad_scale, int zero_grad, void* stream) {
  if (n <= 0) return 0;
  sgd_momentum_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(
      (float*)param, (float*)grad, (float*)mom, n, lr, momentum, weight_decay, grad_scale,
      zero_grad);
  return (int)cudaGetLastError();
}

}  // extern "C"
