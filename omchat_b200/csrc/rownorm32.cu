// Row kernels of decoders whose residual stream is fp32: scaled embedding gather, RMS norm of fp32 rows, and the
// output-side norm + residual add (x <- x + y / rms(y) * (1 + g)) that also emits the rounded copy the next sublayer reads.
// One CTA per row; the row is read once into registers / shared memory, the statistics are fp32. HBM-bound row work.
#include "seq_common.cuh"

namespace omc {

template <typename TT, typename TB>
__global__ void __launch_bounds__(256) embed_scale_kernel(const int32_t* __restrict__ ids, const TT* __restrict__ table, int C,
                                                          int vocab, float scale, float* __restrict__ h32, long long ldh,
                                                          TB* __restrict__ xb, long long ldxb) {
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = ok ? ldf(table + (long long)id * C + c) * scale : 0.f;
    h32[(long long)t * ldh + c] = v;
    if (xb != nullptr) stf(xb + (long long)t * ldxb + c, v);
  }
}

// Embedding row plus the sinusoidal position vector: entry 2i is sin(p * f_i), entry 2i + 1 is cos(p * f_i). The angle is formed
// and reduced in double precision (f_i arrives as a double table), so it is exact to fp32 at any position.
template <typename TT>
__global__ void __launch_bounds__(256) embed_sinusoid_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ pos,
                                                             const TT* __restrict__ table, int C, int vocab, float scale,
                                                             const double* __restrict__ freq, float* __restrict__ h32, long long ldh) {
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  const double p = (double)pos[t];
  for (int i = threadIdx.x; 2 * i < C; i += blockDim.x) {
    double sn, cs;
    sincos(p * freq[i], &sn, &cs);
    const int c = 2 * i;
    h32[(long long)t * ldh + c] = (ok ? ldf(table + (long long)id * C + c) * scale : 0.f) + (float)sn;
    if (c + 1 < C) h32[(long long)t * ldh + c + 1] = (ok ? ldf(table + (long long)id * C + c + 1) * scale : 0.f) + (float)cs;
  }
}

template <typename TW, typename TY>
__global__ void __launch_bounds__(256) rms_rows_kernel(const float* __restrict__ x, long long ldx, const TW* __restrict__ w,
                                                       int one_plus, float eps, TY* __restrict__ y, long long ldy, int n) {
  __shared__ float red[33];
  const float* xr = x + (long long)blockIdx.x * ldx;
  float ss = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = xr[c];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)n + eps);
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    float g = 1.f;
    if (w != nullptr) g = one_plus ? 1.f + ldf(w + c) : ldf(w + c);
    stf(y + (long long)blockIdx.x * ldy + c, xr[c] * rstd * g);
  }
}

template <typename TW, typename TB>
__global__ void __launch_bounds__(256) norm_residual_kernel(const float* __restrict__ y, long long ldy, const TW* __restrict__ w,
                                                            float eps, float* __restrict__ h32, long long ldh,
                                                            TB* __restrict__ xb, long long ldxb, int C) {
  __shared__ float red[33];
  const float* yr = y + (long long)blockIdx.x * ldy;
  float ss = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = yr[c];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)C + eps);
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = h32[(long long)blockIdx.x * ldh + c] + yr[c] * rstd * (1.f + ldf(w + c));
    h32[(long long)blockIdx.x * ldh + c] = v;
    if (xb != nullptr) stf(xb + (long long)blockIdx.x * ldxb + c, v);
  }
}


// Sublayer output -> residual stream -> next sublayer's input, one CTA per row, the row staged in shared memory:
//   y = y1                                               (y2 == NULL)
//   y = (y1 / rms(y1) * wa + y2 / rms(y2) * wb) / 2      (two mixers side by side, each normed with a plain weight first)
//   h32 += mult * y / rms(y) * (1 + w_post)
//   xb = h32 / rms(h32) * (1 + w_next)   (w_next == NULL: xb = round(h32); xb == NULL: nothing)
template <typename TW, typename TB>
__global__ void __launch_bounds__(256) post_norm_residual_kernel(const float* __restrict__ y1, long long ld1, const TW* __restrict__ wa,
                                                                 const float* __restrict__ y2, long long ld2, const TW* __restrict__ wb,
                                                                 const TW* __restrict__ w_post, float eps, float mult,
                                                                 float* __restrict__ h32, long long ldh, const TW* __restrict__ w_next,
                                                                 TB* __restrict__ xb, long long ldxb, int C) {
  extern __shared__ float row[];  // [C]
  __shared__ float red[33];
  const long long t = blockIdx.x;
  float s1 = 0.f, s2 = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float a = y1[t * ld1 + c];
    s1 = fmaf(a, a, s1);
    if (y2 != nullptr) {
      const float b = y2[t * ld2 + c];
      s2 = fmaf(b, b, s2);
    }
  }
  s1 = block_sum(s1, red);
  float ss = 0.f;
  if (y2 != nullptr) {
    s2 = block_sum(s2, red);
    const float r1 = 1.f / sqrtf(s1 / (float)C + eps), r2 = 1.f / sqrtf(s2 / (float)C + eps);
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      const float v = 0.5f * (y1[t * ld1 + c] * r1 * ldf(wa + c) + y2[t * ld2 + c] * r2 * ldf(wb + c));
      row[c] = v;
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
  } else {
    for (int c = threadIdx.x; c < C; c += blockDim.x) row[c] = y1[t * ld1 + c];
    ss = s1;
  }
  const float rstd = 1.f / sqrtf(ss / (float)C + eps);
  float sh = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {   // every thread rereads only what it wrote
    const float v = h32[t * ldh + c] + mult * (row[c] * rstd * (1.f + ldf(w_post + c)));
    h32[t * ldh + c] = v;
    row[c] = v;
    sh = fmaf(v, v, sh);
  }
  if (xb == nullptr) return;
  if (w_next == nullptr) {
    for (int c = threadIdx.x; c < C; c += blockDim.x) stf(xb + t * ldxb + c, row[c]);
    return;
  }
  sh = block_sum(sh, red);
  const float rn = 1.f / sqrtf(sh / (float)C + eps);
  for (int c = threadIdx.x; c < C; c += blockDim.x) stf(xb + t * ldxb + c, row[c] * rn * (1.f + ldf(w_next + c)));
}

// out = act(gate) * up over the two halves of a stacked projection: z [rows, 2 * n] -> out [rows, n]; the arithmetic is fp32.
// Four neighbouring columns per thread (8- or 16-byte accesses) when the rows are laid out for it, else one.
__device__ __forceinline__ void ld4(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
}
__device__ __forceinline__ void ld4(const bf16_t* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
  v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
}
__device__ __forceinline__ void st4(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void st4(bf16_t* p, const float (&v)[4]) {
  uint2 t;
  *reinterpret_cast<__nv_bfloat162*>(&t.x) = __floats2bfloat162_rn(v[0], v[1]);
  *reinterpret_cast<__nv_bfloat162*>(&t.y) = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = t;
}
struct GluParams {
  int act;
  float limit, slope, shift;   // OMC_ACT_CLAMP_SWISH only
};
__device__ __forceinline__ float glu_pair(float g, float u, const GluParams& p) {
  if (p.act == OMC_ACT_CLAMP_SWISH) {
    g = fminf(g, p.limit);
    u = fminf(fmaxf(u, -p.limit), p.limit);
    return g / (1.f + expf(-p.slope * g)) * (u + p.shift);
  }
  if (p.act == OMC_ACT_GELU_TANH) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
  if (p.act == OMC_ACT_GELU_ERF) return 0.5f * g * (1.f + erff(g * 0.70710678118654752f)) * u;
  if (p.act == OMC_ACT_RELU2) return fmaxf(g, 0.f) * fmaxf(g, 0.f) * u;
  if (p.act == OMC_ACT_SILU) return g / (1.f + expf(-g)) * u;
  return g * u;
}

template <typename TZ, typename TY, int VEC>
__global__ void __launch_bounds__(256) glu_mul_kernel(const TZ* __restrict__ z, long long ldz, int n, GluParams gp, TY* __restrict__ y,
                                                      long long ldy, long long total) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // one thread per VEC columns
  if (e >= total) return;
  const int per_row = n / VEC;
  const long long t = e / per_row;
  const int c = (int)(e - t * per_row) * VEC;
  if (VEC == 4) {
    float g[4], u[4];
    ld4(z + t * ldz + c, g);
    ld4(z + t * ldz + n + c, u);
#pragma unroll
    for (int i = 0; i < 4; ++i) g[i] = glu_pair(g[i], u[i], gp);
    st4(y + t * ldy + c, g);
  } else {
    stf(y + t * ldy + c, glu_pair(ldf(z + t * ldz + c), ldf(z + t * ldz + n + c), gp));
  }
}


// y[t, c] = tanh(alpha * x[t, c]) * w[c] + b[c]: a norm without statistics (alpha one scalar in device memory).
template <typename TW, typename TY>
__global__ void __launch_bounds__(256) dyt_rows_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ alpha_p,
                                                       const TW* __restrict__ w, const TW* __restrict__ b, TY* __restrict__ y, long long ldy,
                                                       int C, long long total) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const long long t = e / C;
  const int c = (int)(e - t * C);
  stf(y + t * ldy + c, fmaf(tanhf(*alpha_p * x[t * ldx + c]), ldf(w + c), ldf(b + c)));
}

// x[t, c] <- cap * tanh(x[t, c] / cap), in place.
__global__ void __launch_bounds__(256) tanh_cap_rows_kernel(float* __restrict__ x, long long ldx, int cols, long long total, float cap) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const long long t = e / cols;
  float* p = x + t * ldx + (e - t * cols);
  *p = cap * tanhf(*p / cap);
}

}  // namespace omc

using namespace omc;

extern "C" int omc_embed_scale(const int32_t* ids, int T, const void* table, int t_dt, int C, int vocab, float scale, float* h32,
                               long long ldh, void* xb, int xb_dt, long long ldxb, void* stream) {
  if (ids == nullptr || table == nullptr || h32 == nullptr || T < 0 || C <= 0) return set_error(OMC_ERR_ARG, "omc_embed_scale: bad argument");
  if (T == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(t_dt, TT, OMC_DT_SWITCH(xb_dt, TB, {
    embed_scale_kernel<TT, TB><<<T, 256, 0, st>>>(ids, static_cast<const TT*>(table), C, vocab, scale, h32, ldh,
                                                   static_cast<TB*>(xb), ldxb);
  }))
  return check_launch("omc_embed_scale");
}

extern "C" int omc_rms_rows(const float* x, long long ldx, const void* w, int w_dt, int one_plus, float eps, void* y, int y_dt,
                            long long ldy, int rows, int n, void* stream) {
  if (x == nullptr || y == nullptr || rows < 0 || n <= 0) return set_error(OMC_ERR_ARG, "omc_rms_rows: bad argument");
  if (rows == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(w_dt, TW, OMC_DT_SWITCH(y_dt, TY, {
    rms_rows_kernel<TW, TY><<<rows, 256, 0, st>>>(x, ldx, static_cast<const TW*>(w), one_plus, eps, static_cast<TY*>(y), ldy, n);
  }))
  return check_launch("omc_rms_rows");
}

extern "C" int omc_norm_residual(const float* y, long long ldy, const void* w, int w_dt, float eps, float* h32, long long ldh,
                                 void* xb, int xb_dt, long long ldxb, int rows, int C, void* stream) {
  if (y == nullptr || w == nullptr || h32 == nullptr || rows < 0 || C <= 0) return set_error(OMC_ERR_ARG, "omc_norm_residual: bad argument");
  if (rows == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(w_dt, TW, OMC_DT_SWITCH(xb_dt, TB, {
    norm_residual_kernel<TW, TB><<<rows, 256, 0, st>>>(y, ldy, static_cast<const TW*>(w), eps, h32, ldh, static_cast<TB*>(xb), ldxb, C);
  }))
  return check_launch("omc_norm_residual");
}

extern "C" int omc_post_norm_residual(const float* y1, long long ld1, const void* wa, const float* y2, long long ld2, const void* wb,
                                      const void* w_post, int w_dt, float eps, float mult, float* h32, long long ldh,
                                      const void* w_next, void* xb, int xb_dt, long long ldxb, int rows, int C, void* stream) {
  if (y1 == nullptr || w_post == nullptr || h32 == nullptr || rows < 0 || C <= 0 || (y2 != nullptr && (wa == nullptr || wb == nullptr)))
    return set_error(OMC_ERR_ARG, "omc_post_norm_residual: bad argument");
  if (rows == 0) return OMC_OK;
  const size_t smem = (size_t)C * sizeof(float);
  if (smem > 200 * 1024) return set_error(OMC_ERR_SHAPE, "omc_post_norm_residual: row too wide for shared memory");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(w_dt, TW, OMC_DT_SWITCH(xb_dt, TB, {
    if (smem > 48 * 1024) cudaFuncSetAttribute(post_norm_residual_kernel<TW, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    post_norm_residual_kernel<TW, TB><<<rows, 256, smem, st>>>(y1, ld1, static_cast<const TW*>(wa), y2, ld2, static_cast<const TW*>(wb),
                                                               static_cast<const TW*>(w_post), eps, mult, h32, ldh,
                                                               static_cast<const TW*>(w_next), static_cast<TB*>(xb), ldxb, C);
  }))
  return check_launch("omc_post_norm_residual");
}

extern "C" int omc_glu_mul(const void* z, int z_dt, long long ldz, int rows, int n, int act, float limit, float slope, float shift,
                           void* y, int y_dt, long long ldy, void* stream) {
  if (z == nullptr || y == nullptr || rows < 0 || n <= 0) return set_error(OMC_ERR_ARG, "omc_glu_mul: bad argument");
  if (rows == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long total = (long long)rows * n;
  const bool vec = n % 4 == 0 && ldz % 4 == 0 && ldy % 4 == 0 && reinterpret_cast<uintptr_t>(z) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0;
  const GluParams gp{act, limit, slope, shift};
  OMC_DT_SWITCH(z_dt, TZ, OMC_DT_SWITCH(y_dt, TY, {
    if (vec) glu_mul_kernel<TZ, TY, 4><<<(unsigned)((total / 4 + 255) / 256), 256, 0, st>>>(static_cast<const TZ*>(z), ldz, n, gp, static_cast<TY*>(y), ldy, total / 4);
    else glu_mul_kernel<TZ, TY, 1><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(static_cast<const TZ*>(z), ldz, n, gp, static_cast<TY*>(y), ldy, total);
  }))
  return check_launch("omc_glu_mul");
}

extern "C" int omc_embed_sinusoid(const int32_t* ids, const int32_t* pos, int T, const void* table, int t_dt, int C, int vocab, float scale,
                                  const double* freq, float* h32, long long ldh, void* stream) {
  if (ids == nullptr || pos == nullptr || table == nullptr || freq == nullptr || h32 == nullptr || T < 0 || C <= 0)
    return set_error(OMC_ERR_ARG, "omc_embed_sinusoid: bad argument");
  if (T == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(t_dt, TT, {
    embed_sinusoid_kernel<TT><<<T, 256, 0, st>>>(ids, pos, static_cast<const TT*>(table), C, vocab, scale, freq, h32, ldh);
  })
  return check_launch("omc_embed_sinusoid");
}

extern "C" int omc_dyt_rows(const float* x, long long ldx, const float* alpha, const void* w, const void* b, int w_dt, void* y, int y_dt,
                            long long ldy, int rows, int C, void* stream) {
  if (x == nullptr || alpha == nullptr || w == nullptr || b == nullptr || y == nullptr || rows < 0 || C <= 0)
    return set_error(OMC_ERR_ARG, "omc_dyt_rows: bad argument");
  if (rows == 0) return OMC_OK;
  const long long total = (long long)rows * C;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(w_dt, TW, OMC_DT_SWITCH(y_dt, TY, {
    dyt_rows_kernel<TW, TY><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(x, ldx, alpha, static_cast<const TW*>(w), static_cast<const TW*>(b),
                                                                            static_cast<TY*>(y), ldy, C, total);
  }))
  return check_launch("omc_dyt_rows");
}

extern "C" int omc_tanh_cap_rows(float* x, long long ldx, int rows, int cols, float cap, void* stream) {
  if (x == nullptr || rows < 0 || cols <= 0 || !(cap > 0.f)) return set_error(OMC_ERR_ARG, "omc_tanh_cap_rows: bad argument");
  if (rows == 0) return OMC_OK;
  const long long total = (long long)rows * cols;
  tanh_cap_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, ldx, cols, total, cap);
  return check_launch("omc_tanh_cap_rows");
}
