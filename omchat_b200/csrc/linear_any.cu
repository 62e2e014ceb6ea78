// Linear layer for any shape and for fp32 as well as bf16 storage: Y = act(alpha * X W^T), fp32 accumulation on the FMA pipe.
//
// This is the kernel a new decoder is brought up on, the true-fp32 path of the sequence-step models (no reduced-precision
// matrix mode anywhere), and the path for shapes the tcgen05 GEMM does not take (dimensions that are not multiples of 8, head
// slices of a few dozen columns). 64 x 64 output tile per CTA, 256 threads with 4 x 4 outputs each, K walked in slices of 16
// through shared memory (operands converted to fp32 when they are staged). blockIdx.z walks a batch of independent problems
// that are column slices of the same buffers (attention heads); an optional tile -> group table turns it into the grouped
// product of expert-sorted rows. Each output accumulates its K terms in ascending order, whatever the M of the call.
#include "seq_common.cuh"

namespace omc {

constexpr int kLinBM = 64, kLinBN = 64, kLinBK = 16;

struct LinearArgs {
  const void* X;
  const void* W;
  void* Y;
  long long ldx, sx, ldw, sw, ldy, sy, group_stride;
  const int32_t* tile_group;
  int M, N, K;
  float alpha;
  int act;
  const void* bias;  // [N] of the weights' dtype, added before the activation (NULL: none); batch item b reads bias + b * sbias
  long long sbias;
};

__device__ __forceinline__ float apply_act(float z, int act) {
  if (act == OMC_ACT_RELU2) {
    z = fmaxf(z, 0.f);
    return z * z;
  }
  if (act == OMC_ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  if (act == OMC_ACT_GELU_ERF) return 0.5f * z * (1.f + erff(z * 0.70710678118654752f));
  return z;
}

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256) linear_tile_kernel(LinearArgs a) {
  __shared__ float xs[kLinBK][kLinBM + 4];
  __shared__ float ws[kLinBK][kLinBN + 4];
  const int m0 = blockIdx.y * kLinBM, n0 = blockIdx.x * kLinBN;
  const TX* X = static_cast<const TX*>(a.X) + (long long)blockIdx.z * a.sx;
  const TW* W = static_cast<const TW*>(a.W) + (long long)blockIdx.z * a.sw;
  TY* Y = static_cast<TY*>(a.Y) + (long long)blockIdx.z * a.sy;
  if (a.tile_group != nullptr) {
    const int g = a.tile_group[blockIdx.y];
    if (g < 0) return;
    W += (long long)g * a.group_stride;
  }
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  // staging: thread -> (row = tid / 4, k quarter = tid % 4): 4 consecutive k of one row
  const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < a.K; k0 += kLinBK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int m = m0 + lr, n = n0 + lr;
      xs[lk + j][lr] = (m < a.M && k < a.K) ? ldf(X + (long long)m * a.ldx + k) : 0.f;
      ws[lk + j][lr] = (n < a.N && k < a.K) ? ldf(W + (long long)n * a.ldw + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kLinBK; ++k) {
      const float4 xv = *reinterpret_cast<const float4*>(&xs[k][ty * 4]);
      const float4 wv = *reinterpret_cast<const float4*>(&ws[k][tx * 4]);
      const float xr[4] = {xv.x, xv.y, xv.z, xv.w}, wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xr[i], wr[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= a.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < a.N) stf(Y + (long long)m * a.ldy + n, apply_act(acc[i][j] * a.alpha + (a.bias != nullptr ? ldf(static_cast<const TW*>(a.bias) + blockIdx.z * a.sbias + n) : 0.f), a.act));
    }
  }
}

// ---- a few outputs per row (routers, gates, low-rank factors): the tile kernels would leave such a product to a handful of CTAs
// that each walk all of K. Here a CTA takes 8 rows and walks K in chunks of 1024 that it holds in shared memory as fp32; a warp owns
// up to 8 output columns (n = blockIdx.y * 8 + warp, then in strides of 8 * gridDim.y) with 8 accumulators each: it reads a chunk of
// that row of W once for all 8 rows. A lane takes four consecutive k at a time (one 8- or 16-byte load of W, float4 reads of the
// rows), the warp strides the chunk by 128, and a shuffle tree finishes the sums - the order of a sum depends on K alone, with or
// without the vector loads and however the columns are spread over CTAs (all columns in one CTA for long steps, eight per CTA for
// steps of a few rows, where there are few row blocks to fill the device with).
constexpr int kNarrowRows = 8, kNarrowMaxN = 64, kNarrowKC = 1024, kNarrowPerWarp = kNarrowMaxN / 8;

__device__ __forceinline__ void nld4(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
}
__device__ __forceinline__ void nld4(const bf16_t* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x)), hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
  v[0] = lo.x, v[1] = lo.y, v[2] = hi.x, v[3] = hi.y;
}

template <typename TX, typename TW, typename TY, bool VEC>
__global__ void __launch_bounds__(256, 2) linear_narrow_kernel(LinearArgs a) {
  __shared__ __align__(16) float nxs[kNarrowRows][kNarrowKC];
  const int m0 = blockIdx.x * kNarrowRows, nr = min(kNarrowRows, a.M - m0);
  const TX* X = static_cast<const TX*>(a.X) + (long long)blockIdx.z * a.sx;
  const TW* W = static_cast<const TW*>(a.W) + (long long)blockIdx.z * a.sw;
  TY* Y = static_cast<TY*>(a.Y) + (long long)blockIdx.z * a.sy;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.y * 8 + warp, stride = 8 * gridDim.y;
  float acc[kNarrowPerWarp][kNarrowRows];
#pragma unroll
  for (int i = 0; i < kNarrowPerWarp; ++i)
#pragma unroll
    for (int r = 0; r < kNarrowRows; ++r) acc[i][r] = 0.f;
  for (int kc = 0; kc < a.K; kc += kNarrowKC) {
    const int kn = min(kNarrowKC, a.K - kc), knp = (kn + 3) & ~3;   // the chunk's columns, rounded up to 4 with a zero tail
    if (kc > 0) __syncthreads();
    if (VEC) {
      const int k4n = knp >> 2;
      for (int e = threadIdx.x; e < kNarrowRows * k4n; e += blockDim.x) {
        const int r = e / k4n, k = (e - r * k4n) << 2;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (r < nr) nld4(X + (long long)(m0 + r) * a.ldx + kc + k, v);
        *reinterpret_cast<float4*>(&nxs[r][k]) = make_float4(v[0], v[1], v[2], v[3]);
      }
    } else {
      for (int e = threadIdx.x; e < kNarrowRows * knp; e += blockDim.x) {
        const int r = e / knp, k = e - r * knp;
        nxs[r][k] = (r < nr && k < kn) ? ldf(X + (long long)(m0 + r) * a.ldx + kc + k) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kNarrowPerWarp; ++i) {
      const int n = n0 + i * stride;
      if (n < a.N) {
        const TW* wr = W + (long long)n * a.ldw + kc;
#pragma unroll 2
        for (int k = lane * 4; k < knp; k += 128) {
          float wv[4];
          if (VEC) {
            nld4(wr + k, wv);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = k + j < kn ? ldf(wr + k + j) : 0.f;
          }
#pragma unroll
          for (int r = 0; r < kNarrowRows; ++r) {
            const float4 xv = *reinterpret_cast<const float4*>(&nxs[r][k]);
            acc[i][r] = fmaf(xv.x, wv[0], acc[i][r]);
            acc[i][r] = fmaf(xv.y, wv[1], acc[i][r]);
            acc[i][r] = fmaf(xv.z, wv[2], acc[i][r]);
            acc[i][r] = fmaf(xv.w, wv[3], acc[i][r]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kNarrowPerWarp; ++i) {
    const int n = n0 + i * stride;
    if (n >= a.N) break;
    float mine = 0.f;
#pragma unroll
    for (int r = 0; r < kNarrowRows; ++r) {
      const float v = seq_warp_sum(acc[i][r]);
      if (lane == r) mine = v;
    }
    if (lane < nr) {
      const float b = a.bias != nullptr ? ldf(static_cast<const TW*>(a.bias) + blockIdx.z * a.sbias + n) : 0.f;
      stf(Y + (long long)(m0 + lane) * a.ldy + n, apply_act(mine * a.alpha + b, a.act));
    }
  }
}

// ---- bf16 x bf16 on the tensor pipe (mma.sync.m16n8k16): the same interface for operands whose rows start on 16-byte boundaries.
// 128 x 128 output tile, K slices of 32 double-buffered with cp.async, 8 warps of 64 x 32. It serves the batched per-head products
// of latent attention (absorbing W_uk into the query, W_uv after the attention), whose heads are column slices of one buffer.
constexpr int kMmaBM = 128, kMmaBN = 128, kMmaBK = 32, kMmaPitch = kMmaBK + 8;

__device__ __forceinline__ uint32_t lin_smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void store_pair(float* p, float x, float y) { *reinterpret_cast<float2*>(p) = make_float2(x, y); }
__device__ __forceinline__ void store_pair(bf16_t* p, float x, float y) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(x, y); }

template <typename TY>
__global__ void __launch_bounds__(256) linear_mma_kernel(LinearArgs a) {
  __shared__ __align__(16) bf16_t As[2][kMmaBM * kMmaPitch];
  __shared__ __align__(16) bf16_t Bs[2][kMmaBN * kMmaPitch];
  const int m0 = blockIdx.y * kMmaBM, n0 = blockIdx.x * kMmaBN;
  const bf16_t* X = static_cast<const bf16_t*>(a.X) + (long long)blockIdx.z * a.sx;
  const bf16_t* W = static_cast<const bf16_t*>(a.W) + (long long)blockIdx.z * a.sw;
  TY* Y = static_cast<TY*>(a.Y) + (long long)blockIdx.z * a.sy;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp >> 2, wn = warp & 3;  // 2 x 4 warps: rows wm * 64, columns wn * 32
  float acc[4][4][4] = {};
  auto stage = [&](int buf, int k0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + i * 256;          // 512 chunks of 8 elements per operand tile
      const int row = idx >> 2, c = (idx & 3) * 8;
      const int k = k0 + c;
      bf16_t* da = &As[buf][row * kMmaPitch + c];
      bf16_t* db = &Bs[buf][row * kMmaPitch + c];
      if (m0 + row < a.M && k < a.K)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(lin_smem_u32(da)), "l"(X + (long long)(m0 + row) * a.ldx + k));
      else *reinterpret_cast<uint4*>(da) = make_uint4(0, 0, 0, 0);
      if (n0 + row < a.N && k < a.K)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(lin_smem_u32(db)), "l"(W + (long long)(n0 + row) * a.ldw + k));
      else *reinterpret_cast<uint4*>(db) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int nk = (a.K + kMmaBK - 1) / kMmaBK;
  stage(0, 0);
  for (int kt = 0; kt < nk; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < nk) {
      stage(buf ^ 1, (kt + 1) * kMmaBK);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kMmaBK; kk += 16) {
      uint32_t bfr[4][2];
#pragma unroll
      for (int nn = 0; nn < 2; ++nn) {  // two 8-column tiles per ldmatrix.x4
        const bf16_t* pb = &Bs[buf][(wn * 32 + nn * 16 + (lane & 7) + 8 * (lane >> 4)) * kMmaPitch + kk + 8 * ((lane >> 3) & 1)];
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(bfr[2 * nn][0]), "=r"(bfr[2 * nn][1]), "=r"(bfr[2 * nn + 1][0]), "=r"(bfr[2 * nn + 1][1])
                     : "r"(lin_smem_u32(pb)));
      }
#pragma unroll
      for (int mm = 0; mm < 4; ++mm) {
        uint32_t a0, a1, a2, a3;
        const bf16_t* pa = &As[buf][(wm * 64 + mm * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * kMmaPitch + kk + 8 * (lane >> 4)];
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(lin_smem_u32(pa)));
#pragma unroll
        for (int nn = 0; nn < 4; ++nn)
          asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                       : "+f"(acc[mm][nn][0]), "+f"(acc[mm][nn][1]), "+f"(acc[mm][nn][2]), "+f"(acc[mm][nn][3])
                       : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(bfr[nn][0]), "r"(bfr[nn][1]));
      }
    }
    __syncthreads();
  }
  const int g = lane >> 2, t4 = lane & 3;
  // an accumulator pair (columns n, n + 1) goes out as one 4- or 8-byte store when the row is laid out for it
  const bool pair_ok = (a.ldy % 2 == 0) && (a.sy % 2 == 0) && (reinterpret_cast<uintptr_t>(a.Y) % (2 * sizeof(TY)) == 0);
#pragma unroll
  for (int mm = 0; mm < 4; ++mm)
#pragma unroll
    for (int nn = 0; nn < 4; ++nn)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int m = m0 + wm * 64 + mm * 16 + g + 8 * hh;
        const int n = n0 + wn * 32 + nn * 8 + 2 * t4;
        if (m >= a.M || n >= a.N) continue;
        const bf16_t* bias = a.bias != nullptr ? static_cast<const bf16_t*>(a.bias) + blockIdx.z * a.sbias : nullptr;
        const float b0 = bias != nullptr ? ldf(bias + n) : 0.f, b1 = (bias != nullptr && n + 1 < a.N) ? ldf(bias + n + 1) : 0.f;
        const float v0 = apply_act(acc[mm][nn][2 * hh] * a.alpha + b0, a.act), v1 = apply_act(acc[mm][nn][2 * hh + 1] * a.alpha + b1, a.act);
        TY* dst = Y + (long long)m * a.ldy + n;
        if (pair_ok && n + 1 < a.N) {
          store_pair(dst, v0, v1);
        } else {
          stf(dst, v0);
          if (n + 1 < a.N) stf(dst + 1, v1);
        }
      }
}

static bool mma_operands_ok(const LinearArgs& a) {
  return a.tile_group == nullptr && a.K % 8 == 0 && a.ldx % 8 == 0 && a.ldw % 8 == 0 && a.sx % 8 == 0 && a.sw % 8 == 0 &&
         reinterpret_cast<uintptr_t>(a.X) % 16 == 0 && reinterpret_cast<uintptr_t>(a.W) % 16 == 0;
}

static int launch_linear_mma(const LinearArgs& a, int y_dt, int batch, cudaStream_t st) {
  dim3 grid((a.N + kMmaBN - 1) / kMmaBN, (a.M + kMmaBM - 1) / kMmaBM, batch);
  if (y_dt == OMC_DT_F32) linear_mma_kernel<float><<<grid, 256, 0, st>>>(a);
  else if (y_dt == OMC_DT_BF16) linear_mma_kernel<bf16_t><<<grid, 256, 0, st>>>(a);
  else return set_error(OMC_ERR_ARG, "omc_linear: unknown output dtype");
  return check_launch("omc_linear");
}

template <typename TX, typename TW, typename TY>
static int launch_narrow_typed(const LinearArgs& a, int batch, cudaStream_t st) {
  // vector loads: rows of X and W that start on 8-byte (bf16) / 16-byte (fp32) boundaries and a K that is a multiple of four
  const bool vec = a.K % 4 == 0 && a.ldx % 4 == 0 && a.ldw % 4 == 0 && a.sx % 4 == 0 && a.sw % 4 == 0 &&
                   reinterpret_cast<uintptr_t>(a.X) % (4 * sizeof(TX)) == 0 && reinterpret_cast<uintptr_t>(a.W) % (4 * sizeof(TW)) == 0;
  // where the columns run is a matter of occupancy only: every column is summed by one warp in the same order either way
  const dim3 grid((a.M + kNarrowRows - 1) / kNarrowRows, a.M <= 64 ? (a.N + 7) / 8 : 1, batch);
  if (vec) linear_narrow_kernel<TX, TW, TY, true><<<grid, 256, 0, st>>>(a);
  else linear_narrow_kernel<TX, TW, TY, false><<<grid, 256, 0, st>>>(a);
  return check_launch("omc_linear");
}

template <typename TX, typename TW>
static int launch_narrow(const LinearArgs& a, int y_dt, int batch, cudaStream_t st) {
  if (y_dt == OMC_DT_F32) return launch_narrow_typed<TX, TW, float>(a, batch, st);
  if (y_dt == OMC_DT_BF16) return launch_narrow_typed<TX, TW, bf16_t>(a, batch, st);
  return set_error(OMC_ERR_ARG, "omc_linear: unknown output dtype");
}

template <typename TX, typename TW>
static int launch_linear(const LinearArgs& a, int y_dt, int batch, cudaStream_t st) {
  // few outputs over a long K: the choice depends on widths only, never on M
  if (a.tile_group == nullptr && a.N <= kNarrowMaxN && a.K >= 4 * a.N) return launch_narrow<TX, TW>(a, y_dt, batch, st);
  dim3 grid((a.N + kLinBN - 1) / kLinBN, (a.M + kLinBM - 1) / kLinBM, batch);
  if (y_dt == OMC_DT_F32) linear_tile_kernel<TX, TW, float><<<grid, 256, 0, st>>>(a);
  else if (y_dt == OMC_DT_BF16) linear_tile_kernel<TX, TW, bf16_t><<<grid, 256, 0, st>>>(a);
  else return set_error(OMC_ERR_ARG, "omc_linear: unknown output dtype");
  return check_launch("omc_linear");
}

}  // namespace omc

extern "C" int omc_linear_bias(const void* X, int x_dt, long long ldx, long long sx, const void* W, int w_dt, long long ldw,
                               long long sw, void* Y, int y_dt, long long ldy, long long sy, int M, int N, int K, int batch,
                               float alpha, int act, const int32_t* tile_group, long long group_stride, const void* bias,
                               long long sbias, void* stream) {
  using namespace omc;
  if (X == nullptr || W == nullptr || Y == nullptr || N <= 0 || K <= 0 || M < 0 || batch <= 0)
    return set_error(OMC_ERR_ARG, "omc_linear: bad argument");
  if (M == 0) return OMC_OK;
  if (tile_group != nullptr && batch != 1) return set_error(OMC_ERR_ARG, "omc_linear: a tile table excludes a batch");
  if ((long long)((M + kLinBM - 1) / kLinBM) > 65535 || batch > 65535)
    return set_error(OMC_ERR_SHAPE, "omc_linear: more than 65535 row tiles or batch items");
  if (bias != nullptr && tile_group != nullptr) return set_error(OMC_ERR_ARG, "omc_linear: a bias excludes a tile table");
  LinearArgs a{X, W, Y, ldx, sx, ldw, sw, ldy, sy, group_stride, tile_group, M, N, K, alpha, act, bias, sbias};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (x_dt == OMC_DT_F32 && w_dt == OMC_DT_F32) return launch_linear<float, float>(a, y_dt, batch, st);
  if (x_dt == OMC_DT_F32 && w_dt == OMC_DT_BF16) return launch_linear<float, bf16_t>(a, y_dt, batch, st);
  if (x_dt == OMC_DT_BF16 && w_dt == OMC_DT_BF16) {
    // the choice depends on layout and widths only, never on M: a row is computed by the same kernel in every batch
    const bool narrow = tile_group == nullptr && N <= kNarrowMaxN && K >= 4 * N;
    if (!narrow && mma_operands_ok(a) && (long long)N * K >= 4096) return launch_linear_mma(a, y_dt, batch, st);
    return launch_linear<bf16_t, bf16_t>(a, y_dt, batch, st);
  }
  return set_error(OMC_ERR_ARG, "omc_linear: operand dtypes must be (f32, f32), (f32, bf16) or (bf16, bf16)");
}

extern "C" int omc_linear(const void* X, int x_dt, long long ldx, long long sx, const void* W, int w_dt, long long ldw,
                          long long sw, void* Y, int y_dt, long long ldy, long long sy, int M, int N, int K, int batch,
                          float alpha, int act, const int32_t* tile_group, long long group_stride, void* stream) {
  return omc_linear_bias(X, x_dt, ldx, sx, W, w_dt, ldw, sw, Y, y_dt, ldy, sy, M, N, K, batch, alpha, act, tile_group, group_stride,
                         nullptr, 0, stream);
}
