// Sliding-window softmax attention over a paged key/value cache, without rotation: positions enter through a bias that depends on
// the distance between query and key only. Per cached token one row [kv_heads * dim keys | kv_heads * vdim values].
//
//   omc_qk_norm_kv_store: the rows of a step -> normed queries, and normed keys + values appended to the pages (one RMS norm over the
//                         whole projection, or one per group of columns - a head, or a score map of a head - with a shared weight)
//   omc_window_attn:      score = (q . k) * scale -> softcap * tanh(score / softcap) -> + dist_bias[i - j][head] -> softmax over the
//                         keys j with 0 <= i - j < window, and the first keep_first keys of the sequence whatever their distance
//                         -> weighted sum of values. maps > 1: every head has that many score maps (queries and keys of their own)
//                         over the same values; the maps come out side by side.
//   omc_diff_heads_gate:  two maps -> o = a1 - lambda a2, RMS norm over the head, a constant factor, an elementwise gate
// The distance bias arrives as a table [window, heads] that the host builds (here from a bucketed learned table; any function of
// the distance fits). Prompt portions and decoded tokens are one case: row t at position pos[t] of slot[t] reads the cached
// entries max(0, pos - window + 1) .. pos of its slot, which the store kernel of the same step has written.
// The plain kernel: fp32 arithmetic, one CTA per (row, head), a warp per key, lanes across the head dimension.
#include <math.h>

#include "seq_common.cuh"

namespace omc {

constexpr int kWinWarps = 4;
constexpr int kWinMaxPerLane = 8;  // value width up to 256

// One CTA per row. q: RMS norm with a plain weight -> q_out; k likewise -> page; v copied -> page. group 0: one norm over all
// columns, weight [n]; group > 0: one norm per `group` consecutive columns (a warp each), weight [group] shared by the groups.
template <typename TW, typename TD>
__device__ __forceinline__ void rms_to(const float* __restrict__ x, int n, int group, const TW* __restrict__ w, float eps,
                                       TD* __restrict__ dst, float* red) {
  if (group <= 0) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) ss = fmaf(x[c], x[c], ss);
    ss = block_sum(ss, red);
    const float rstd = 1.f / sqrtf(ss / (float)n + eps);
    for (int c = threadIdx.x; c < n; c += blockDim.x) stf(dst + c, x[c] * rstd * ldf(w + c));
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int g = warp; g * group < n; g += nw) {
    const float* xg = x + g * group;
    float ss = 0.f;
    for (int c = lane; c < group; c += 32) ss = fmaf(xg[c], xg[c], ss);
    ss = seq_warp_sum(ss);
    const float rstd = 1.f / sqrtf(ss / (float)group + eps);
    for (int c = lane; c < group; c += 32) stf(dst + g * group + c, xg[c] * rstd * ldf(w + c));
  }
}

template <typename TW, typename TC>
__global__ void __launch_bounds__(256) qk_norm_kv_store_kernel(const float* __restrict__ q, long long ldq, int nq, int q_group,
                                                               const TW* __restrict__ wq, const float* __restrict__ k, long long ldk,
                                                               int nk, int k_group, const TW* __restrict__ wk, const float* __restrict__ v,
                                                               long long ldv, int nv, float eps, const int32_t* __restrict__ pos,
                                                               const int32_t* __restrict__ slot, const int32_t* __restrict__ block_table,
                                                               int max_pages, int page_size, TC* __restrict__ pool,
                                                               TC* __restrict__ q_out, long long ldqo) {
  __shared__ float red[33];
  const long long t = blockIdx.x;
  const int p = pos[t];
  const int page = block_table[(long long)slot[t] * max_pages + p / page_size];
  TC* dst = pool + ((long long)page * page_size + p % page_size) * (nk + nv);
  rms_to(q + t * ldq, nq, q_group, wq, eps, q_out + t * ldqo, red);
  rms_to(k + t * ldk, nk, k_group, wk, eps, dst, red);
  for (int c = threadIdx.x; c < nv; c += blockDim.x) stf(dst + nk + c, v[t * ldv + c]);
}

// Rows of a step for an attention with positions in the queries and keys themselves. Per head: the first rot_dims dimensions of
// queries and keys are rotated pairwise - (u, v) at (2i, 2i + 1) becomes (u cos a - v sin a, v cos a + u sin a), a = position * freq[i],
// the angle formed in fp32 - (freq NULL: no rotation); queries are multiplied by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)
// (temp_coef 0: off); values are divided by their root mean square over each head's dv values when v_unit is set. Queries go to
// q_out, keys and values to the cache row of (slot, position). One CTA per row.
template <typename TC>
__global__ void __launch_bounds__(256) pos_qkv_store_kernel(const float* __restrict__ q, long long ldq, int H, const float* __restrict__ k,
                                                            long long ldk, int G, int d, const float* __restrict__ v, long long ldv, int dv,
                                                            const float* __restrict__ freq, int rot_dims, float temp_coef, int temp_every,
                                                            int v_unit, float eps, const int32_t* __restrict__ pos,
                                                            const int32_t* __restrict__ slot, const int32_t* __restrict__ block_table,
                                                            int max_pages, int page_size, TC* __restrict__ pool, TC* __restrict__ q_out,
                                                            long long ldqo) {
  extern __shared__ float cs[];   // [rot_dims / 2][2]: cos, sin
  const long long t = blockIdx.x;
  const int p = pos[t];
  const int page = block_table[(long long)slot[t] * max_pages + p / page_size];
  const int nk = G * d, nv = G * dv, half = freq != nullptr ? rot_dims / 2 : 0;
  TC* dst = pool + ((long long)page * page_size + p % page_size) * (nk + nv);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float a = (float)p * freq[i];
    cs[2 * i] = cosf(a);
    cs[2 * i + 1] = sinf(a);
  }
  __syncthreads();
  float temp = 1.f;
  if (temp_coef != 0.f) temp = 1.f + temp_coef * logf((float)((p + 1) / temp_every) + 1.f);
  const float* qr = q + t * ldq;
  const float* kr = k + t * ldk;
  // queries then keys: (head, pair) for the rotated part, single elements for the rest
  const int qpairs = H * half, kpairs = G * half;
  for (int e = threadIdx.x; e < qpairs + kpairs; e += blockDim.x) {
    const bool isq = e < qpairs;
    const int ee = isq ? e : e - qpairs, hh = ee / half, i = ee - hh * half;
    const float* src = (isq ? qr : kr) + hh * d + 2 * i;
    const float c = cs[2 * i], sn = cs[2 * i + 1], a0 = src[0], a1 = src[1];
    const float r0 = a0 * c - a1 * sn, r1 = a1 * c + a0 * sn;
    if (isq) {
      stf(q_out + t * ldqo + hh * d + 2 * i, r0 * temp);
      stf(q_out + t * ldqo + hh * d + 2 * i + 1, r1 * temp);
    } else {
      stf(dst + hh * d + 2 * i, r0);
      stf(dst + hh * d + 2 * i + 1, r1);
    }
  }
  const int rest = d - 2 * half;
  for (int e = threadIdx.x; e < (H + G) * rest; e += blockDim.x) {
    const int hh = e / rest, c = 2 * half + (e - hh * rest);
    if (hh < H) stf(q_out + t * ldqo + hh * d + c, qr[hh * d + c] * temp);
    else stf(dst + (hh - H) * d + c, kr[(hh - H) * d + c]);
  }
  const float* vr = v + t * ldv;
  if (!v_unit) {
    for (int c = threadIdx.x; c < nv; c += blockDim.x) stf(dst + nk + c, vr[c]);
  } else {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int g = warp; g < G; g += nw) {
      float ss = 0.f;
      for (int c = lane; c < dv; c += 32) ss = fmaf(vr[g * dv + c], vr[g * dv + c], ss);
      ss = seq_warp_sum(ss);
      const float rstd = 1.f / sqrtf(ss / (float)dv + eps);
      for (int c = lane; c < dv; c += 32) stf(dst + nk + g * dv + c, vr[g * dv + c] * rstd);
    }
  }
}

template <typename TQ, typename TC, typename TY>
__global__ void __launch_bounds__(kWinWarps * 32) window_attn_kernel(const TQ* __restrict__ q, long long ldq, int H, int G, int d,
                                                                     int dv, int maps, const TC* __restrict__ pool,
                                                                     const int32_t* __restrict__ block_table, int max_pages,
                                                                     int page_size, const int32_t* __restrict__ pos,
                                                                     const int32_t* __restrict__ slot, int window, int keep_first,
                                                                     float scale, float softcap, const float* __restrict__ dist_bias,
                                                                     const float* __restrict__ sink, const float* __restrict__ gate,
                                                                     long long ldg, int gate_act, TY* __restrict__ out, long long ldo) {
  extern __shared__ float sm[];  // q [d] | acc [warps][dv] | m [warps] | l [warps]
  // blockIdx.y = head * maps + map: queries and outputs are laid out [head][map][.], keys [key/value head][map][d]
  const int t = blockIdx.x, hm = blockIdx.y, h = hm / maps, mp = hm - h * maps, kvh = h / (H / G);
  float* sq = sm;
  float* sacc = sm + d;
  float* s_m = sacc + kWinWarps * dv;
  float* s_l = s_m + kWinWarps;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c = threadIdx.x; c < d; c += blockDim.x) sq[c] = ldf(q + (long long)t * ldq + hm * d + c);
  __syncthreads();
  const int p = pos[t];
  const int first = max(0, p - window + 1);
  const int kept = min(keep_first, first);   // keys 0 .. kept - 1 lie before the window and are seen all the same
  const int32_t* bt = block_table + (long long)slot[t] * max_pages;
  const int W = G * (maps * d + dv);
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  float m = -INFINITY, l = 0.f;
  float acc[kWinMaxPerLane];
#pragma unroll
  for (int i = 0; i < kWinMaxPerLane; ++i) acc[i] = 0.f;
  // the visible keys in one sequence of indices: 0 .. kept - 1, then first .. p
  const int n_keys = kept + (p - first + 1);
  for (int i = warp; i < n_keys; i += kWinWarps) {
    const int j = i < kept ? i : first + (i - kept);
    const TC* row = pool + ((long long)bt[j / page_size] * page_size + j % page_size) * W;
    const TC* kr = row + (kvh * maps + mp) * d;
    const TC* vr = row + G * maps * d + kvh * dv;
    float s = 0.f;
    for (int c = lane; c < d; c += 32) s = fmaf(sq[c], ldf(kr + c), s);
    s = seq_warp_sum(s) * scale;
    if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);
    if (dist_bias != nullptr && p - j < window) s += dist_bias[(long long)(p - j) * H + h];
    const float mn = fmaxf(m, s);
    const float corr = expf(m - mn), pj = expf(s - mn);  // m = -inf on the first key: corr = 0
    l = l * corr + pj;
#pragma unroll
    for (int i2 = 0; i2 < kWinMaxPerLane; ++i2) {
      const int c = lane + 32 * i2;
      if (c < dv) acc[i2] = acc[i2] * corr + pj * ldf(vr + c);
    }
    m = mn;
  }
#pragma unroll
  for (int i = 0; i < kWinMaxPerLane; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) sacc[warp * dv + c] = acc[i];
  }
  if (lane == 0) {
    s_m[warp] = m;
    s_l[warp] = l;
  }
  __syncthreads();
  // the sink: one more term exp(sink[h]) in the denominator, without a key or a value
  float mt = sink != nullptr ? sink[h] : -INFINITY;
#pragma unroll
  for (int w = 0; w < kWinWarps; ++w) mt = fmaxf(mt, s_m[w]);
  float lt = sink != nullptr ? expf(sink[h] - mt) : 0.f;
  float f[kWinWarps];
#pragma unroll
  for (int w = 0; w < kWinWarps; ++w) {
    f[w] = s_m[w] == -INFINITY ? 0.f : expf(s_m[w] - mt);
    lt += s_l[w] * f[w];
  }
  const float inv = 1.f / lt;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < kWinWarps; ++w) o += sacc[w * dv + c] * f[w];
    o *= inv;
    if (gate != nullptr) {
      const float z = gate[(long long)t * ldg + hm * dv + c];
      o *= gate_act == 1 ? z / (1.f + expf(-z)) : (gate_act == 2 ? 1.f / (1.f + expf(-z)) : z);
    }
    stf(out + (long long)t * ldo + hm * dv + c, o);
  }
}


// ---------------------------------------------------------------------------------------------------------------------------
// Tensor-core kernel (bf16; head widths multiples of 16, values up to 128 wide, heads per key/value head a divisor of 64).
// mma.sync.m16n8k16 over 64-key tiles staged by cp.async straight out of the pages, two buffers. The 64 rows of a tile are
// (token, query head) pairs of ONE key/value head - 64 / (H / G) consecutive tokens of one request - so the heads of a group share
// the staged keys and values. Four warps of 16 rows; S = Q K^T, then scale, soft cap (tanh.approx), distance bias and window
// mask on the accumulators, online softmax in base 2, P (bf16, from the accumulator registers) times V through ldmatrix.trans.
// Work items: int32[4] (first_row, n_tok, slot, first_pos) from the host, or - items == NULL - every row an item of its own,
// read from pos / slot on the device (decode steps, replayable from a CUDA graph).
__device__ __forceinline__ uint32_t wsmem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void w_ldsm_x4(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}
__device__ __forceinline__ void w_ldsm_x4_t(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}
__device__ __forceinline__ void w_mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void w_cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
// tanh(x) = 1 - 2 / (exp(2x) + 1) through the hardware exponential and reciprocal: an absolute error of a few 1e-7, where the
// one-instruction tanh.approx has a relative error of 2^-11 - too coarse for scores, which the soft cap multiplies by tens.
__device__ __forceinline__ float tanh_approx(float x) {
  const float e = exp2f(fminf(x, 20.f) * 2.8853900817779268f);
  return 1.f - __fdividef(2.f, e + 1.f);
}
__device__ __forceinline__ uint32_t w_pack2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void w_st_pair(float* p, float x, float y) { *reinterpret_cast<float2*>(p) = make_float2(x, y); }
__device__ __forceinline__ void w_st_pair(bf16_t* p, float x, float y) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(x, y); }

constexpr int kWmRows = 64, kWmKeys = 64;

struct WinMmaArgs {
  const bf16_t* q;
  long long ldq;
  const bf16_t* pool;
  const int32_t* bt;
  const int32_t* items;   // [n][4] or NULL
  const int32_t* pos;
  const int32_t* slot;
  const float* bias;      // [window][H] or NULL
  const float* sink;      // [H] or NULL: one more term exp(sink[h]) in every softmax denominator
  const float* gate;      // [T][ldg] or NULL: the output is multiplied by act(gate) elementwise
  long long ldg;
  int gate_act;
  void* out;
  long long ldo;
  int max_pages, page_size, H, G, d, dv, window, maps, keep_first;
  float scale, softcap;
  int q_rows;             // rows of the query tile held in shared memory: 64, or the next multiple of 16 above H / G when every item is one token
  int bias_in_smem;       // the bias columns of this key/value head's query heads are staged in shared memory ([window][H / G])
};

template <int NV, typename TO>  // NV: 8-column output tiles, dv <= 8 * NV
__global__ void __launch_bounds__(128) window_attn_mma_kernel(WinMmaArgs a) {
  extern __shared__ __align__(16) unsigned char wsm_raw[];
  const int d = a.d, dv = a.dv, pq = d + 8, pv = dv + 8;
  bf16_t* Qs = reinterpret_cast<bf16_t*>(wsm_raw);
  bf16_t* Ks = Qs + a.q_rows * pq;         // [2][64][pq]
  bf16_t* Vs = Ks + 2 * kWmKeys * pq;      // [2][64][pv]
  float* sbias = reinterpret_cast<float*>(Vs + 2 * kWmKeys * pv);   // [window][rep] when bias_in_smem
  int first_row, n_tok, slot, first_pos;
  if (a.items != nullptr) {
    const int32_t* it = a.items + blockIdx.x * 4;
    first_row = it[0], n_tok = it[1], slot = it[2], first_pos = it[3];
  } else {
    first_row = blockIdx.x, n_tok = 1, slot = a.slot[blockIdx.x], first_pos = a.pos[blockIdx.x];
  }
  const int kvh = blockIdx.y / a.maps, mp = blockIdx.y - kvh * a.maps, rep = a.H / a.G;   // one score map of one key/value head
  const int n_rows = n_tok * rep;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int qchunks = d >> 3, vchunks = dv >> 3;
  for (int i = tid; i < a.q_rows * qchunks; i += blockDim.x) {
    const int row = i / qchunks, c = i - row * qchunks;
    bf16_t* dst = Qs + row * pq + c * 8;
    if (row < n_rows) w_cp_async16(wsmem_u32(dst), a.q + (long long)(first_row + row / rep) * a.ldq + ((kvh * rep + row % rep) * a.maps + mp) * d + c * 8);
    else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
  }
  if (a.bias_in_smem)   // a lookup per score from global memory would be a chain of L2 round trips
    for (int e = tid; e < a.window * rep; e += blockDim.x) sbias[e] = a.bias[(long long)(e / rep) * a.H + kvh * rep + e % rep];
  const int row0 = warp * 16 + g, row1 = row0 + 8;
  const int p0 = row0 < n_rows ? first_pos + row0 / rep : -1, p1 = row1 < n_rows ? first_pos + row1 / rep : -1;   // -1: no such row
  const int h0 = kvh * rep + row0 % rep, h1 = kvh * rep + row1 % rep;
  const int32_t* bt = a.bt + (long long)slot * a.max_pages;
  // key ranges: the kept first keys that lie before the window of the item's first row (none when they touch the window: then
  // the window range simply starts at 0), then the window range up to the item's last row
  int k_begin = max(0, first_pos - a.window + 1);
  const int k_end = first_pos + n_tok;
  int kept_end = min(a.keep_first, k_begin);
  if (kept_end == k_begin) k_begin = 0, kept_end = 0;
  const int kept_tiles = (kept_end + kWmKeys - 1) / kWmKeys, n_tiles = kept_tiles + (k_end - k_begin + kWmKeys - 1) / kWmKeys;
  const int roww = a.G * (a.maps * d + dv);
  // two threads per key: one page lookup per thread and tile, then 16-byte copies at a constant stride
  auto stage = [&](int buf, int tile) {
    const int j0 = tile < kept_tiles ? tile * kWmKeys : k_begin + (tile - kept_tiles) * kWmKeys, j_end = tile < kept_tiles ? kept_end : k_end;
    const int half = tid & 1;
    for (int key = tid >> 1; key < kWmKeys; key += blockDim.x >> 1) {   // one pass with 128 threads, two with the 64 of a one-token item
      const int j = j0 + key;
      bf16_t* kd = Ks + (buf * kWmKeys + key) * pq;
      bf16_t* vd = Vs + (buf * kWmKeys + key) * pv;
      if (j < j_end) {
        const bf16_t* row = a.pool + ((long long)bt[j / a.page_size] * a.page_size + j % a.page_size) * roww;
        const bf16_t* ks = row + (kvh * a.maps + mp) * d;
        const bf16_t* vs = row + a.G * a.maps * d + kvh * dv;
        for (int c = half; c < qchunks; c += 2) w_cp_async16(wsmem_u32(kd + c * 8), ks + c * 8);
        for (int c = half; c < vchunks; c += 2) w_cp_async16(wsmem_u32(vd + c * 8), vs + c * 8);
      } else {
        for (int c = half; c < qchunks; c += 2) *reinterpret_cast<uint4*>(kd + c * 8) = make_uint4(0, 0, 0, 0);
        for (int c = half; c < vchunks; c += 2) *reinterpret_cast<uint4*>(vd + c * 8) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[NV][4];
#pragma unroll
  for (int j = 0; j < NV; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  const int nv = dv >> 3;
  constexpr float kLog2e = 1.4426950408889634f;
  const float inv_cap = a.softcap > 0.f ? 1.f / a.softcap : 0.f;
  stage(0, 0);
  for (int kt = 0; kt < n_tiles; ++kt) {
    const int buf = kt & 1;
    const int j0 = kt < kept_tiles ? kt * kWmKeys : k_begin + (kt - kept_tiles) * kWmKeys, j_end = kt < kept_tiles ? kept_end : k_end;
    if (kt + 1 < n_tiles) {
      stage(buf ^ 1, kt + 1);   // released by the barrier that ended the previous tile
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (warp * 16 < n_rows) {   // a warp without rows (decode: H / G of the 64 rows) only helps staging
      const bf16_t* Kc = Ks + buf * kWmKeys * pq;
      const bf16_t* Vc = Vs + buf * kWmKeys * pv;
      float s[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
      const uint32_t q_base = wsmem_u32(Qs + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * pq + 8 * (lane >> 4));
      const uint32_t k_base = wsmem_u32(Kc + ((lane & 7) + 8 * (lane >> 4)) * pq + 8 * ((lane >> 3) & 1));
      for (int kk = 0; kk < d; kk += 16) {
        uint32_t a0, a1, a2, a3;
        w_ldsm_x4(q_base + kk * 2, a0, a1, a2, a3);
#pragma unroll
        for (int n2 = 0; n2 < 4; ++n2) {
          uint32_t b0, b1, b2, b3;
          w_ldsm_x4(k_base + (n2 * 16 * pq + kk) * 2, b0, b1, b2, b3);
          w_mma_bf16(s[2 * n2], a0, a1, a2, a3, b0, b1);
          w_mma_bf16(s[2 * n2 + 1], a0, a1, a2, a3, b2, b3);
        }
      }
      // scale, soft cap, distance bias, window: scores in base-2 units
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = j0 + n * 8 + 2 * t4 + (e & 1);
          const int p = e < 2 ? p0 : p1, hh = e < 2 ? h0 : h1;
          const int dist = p - key;
          float v = -INFINITY;
          if (key < j_end && dist >= 0 && (dist < a.window || key < a.keep_first)) {
            v = s[n][e] * a.scale;
            if (a.softcap > 0.f) v = a.softcap * tanh_approx(v * inv_cap);
            if (dist < a.window) {   // the table has one row per distance inside the window
              if (a.bias_in_smem) v += sbias[dist * rep + (hh - kvh * rep)];
              else if (a.bias != nullptr) v += __ldg(a.bias + (long long)dist * a.H + hh);
            }
            v *= kLog2e;
          }
          s[n][e] = v;
        }
        mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
        mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;   // rows that see nothing yet
      const float c0 = exp2f(m0 - ms0), c1 = exp2f(m1 - ms1);
      m0 = mn0;
      m1 = mn1;
      float rs0 = 0.f, rs1 = 0.f;
      uint32_t p[8][2];
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        p[n][0] = w_pack2(exp2f(s[n][0] - ms0), exp2f(s[n][1] - ms0));
        p[n][1] = w_pack2(exp2f(s[n][2] - ms1), exp2f(s[n][3] - ms1));
        // the denominator sums the ROUNDED probabilities, the ones the numerator uses
        const float2 f0 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&p[n][0]));
        const float2 f1 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&p[n][1]));
        rs0 += f0.x + f0.y;
        rs1 += f1.x + f1.y;
      }
      l0 = l0 * c0 + rs0;
      l1 = l1 * c1 + rs1;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        o[j][0] *= c0;
        o[j][1] *= c0;
        o[j][2] *= c1;
        o[j][3] *= c1;
      }
      const uint32_t v_base = wsmem_u32(Vc + ((lane & 7) + 8 * ((lane >> 3) & 1)) * pv + 8 * (lane >> 4));
#pragma unroll
      for (int kb16 = 0; kb16 < 4; ++kb16) {
        const uint32_t a0 = p[2 * kb16][0], a1 = p[2 * kb16][1], a2 = p[2 * kb16 + 1][0], a3 = p[2 * kb16 + 1][1];
#pragma unroll
        for (int j = 0; j < NV; j += 2) {
          if (j < nv) {   // dv is a multiple of 16: tiles come in pairs
            uint32_t b0, b1, b2, b3;
            w_ldsm_x4_t(v_base + (kb16 * 16 * pv + j * 8) * 2, b0, b1, b2, b3);
            w_mma_bf16(o[j], a0, a1, a2, a3, b0, b1);
            w_mma_bf16(o[j + 1], a0, a1, a2, a3, b2, b3);
          }
        }
      }
    }
    __syncthreads();   // every warp is done with this tile's buffers
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  float f0 = 1.f, f1 = 1.f;   // factors of the accumulators when the sink moves the reference maximum
  if (a.sink != nullptr) {
    const float s0 = a.sink[h0] * kLog2e, s1 = a.sink[h1] * kLog2e;
    const float r0 = fmaxf(m0, s0), r1 = fmaxf(m1, s1);
    f0 = exp2f(m0 - r0), f1 = exp2f(m1 - r1);
    l0 = l0 * f0 + exp2f(s0 - r0);
    l1 = l1 * f1 + exp2f(s1 - r1);
  }
  const float i0 = f0 / l0, i1 = f1 / l1;
  const long long tr0 = first_row + row0 / rep, tr1 = first_row + row1 / rep;
  TO* out0 = static_cast<TO*>(a.out) + tr0 * a.ldo + (h0 * a.maps + mp) * dv;
  TO* out1 = static_cast<TO*>(a.out) + tr1 * a.ldo + (h1 * a.maps + mp) * dv;
  const float* g0 = a.gate != nullptr ? a.gate + tr0 * a.ldg + (h0 * a.maps + mp) * dv : nullptr;
  const float* g1 = a.gate != nullptr ? a.gate + tr1 * a.ldg + (h1 * a.maps + mp) * dv : nullptr;
  auto gact = [&](float z) { return a.gate_act == 1 ? z / (1.f + __expf(-z)) : (a.gate_act == 2 ? 1.f / (1.f + __expf(-z)) : z); };
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    if (j < nv) {
      const int col = j * 8 + 2 * t4;
      if (row0 < n_rows) {
        float x0 = o[j][0] * i0, x1 = o[j][1] * i0;
        if (g0 != nullptr) x0 *= gact(g0[col]), x1 *= gact(g0[col + 1]);
        w_st_pair(out0 + col, x0, x1);
      }
      if (row1 < n_rows) {
        float x0 = o[j][2] * i1, x1 = o[j][3] * i1;
        if (g1 != nullptr) x0 *= gact(g1[col]), x1 *= gact(g1[col + 1]);
        w_st_pair(out1 + col, x0, x1);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Differential attention of prompt portions in ONE kernel: a CTA takes the 64 (token, query head) rows of one key/value head for BOTH
// score maps. Every 64-key tile is staged once - the two maps' keys and the values they share - and each warp runs the two maps one
// after the other on it (S = Q_m K_m^T, mask, online softmax of its own, P_m V into an accumulator set of its own). The epilogue
// forms o = a1 - lambda a2 on the accumulators, the RMS norm over the head's values (a row's values sit in the four lanes of a
// quad), the constant factor and the elementwise gate, and writes the mixer's pre-projection rows. Compared with one CTA per map and a
// combine kernel behind it: the values travel to shared memory once instead of twice, and the two fp32 maps never travel at all.
struct DiffPairArgs {
  const bf16_t* q;
  long long ldq;
  const bf16_t* pool;
  const int32_t* bt;
  const int32_t* items;   // [n][4] (first_row, n_tok, slot, first_pos)
  const float* gate;      // [T, ldg] or NULL
  long long ldg;
  void* out;              // [T, H * dv]
  long long ldo;
  int max_pages, page_size, H, G, d, dv, window, keep_first, gate_act;
  float scale, lambda, mult, eps;
};

template <int NV, typename TO>
__global__ void __launch_bounds__(128) diff_attn_pair_kernel(DiffPairArgs a) {
  extern __shared__ __align__(16) unsigned char wsm_raw[];
  const int d = a.d, dv = a.dv, pq = d + 8, pv = dv + 8;
  bf16_t* Qs = reinterpret_cast<bf16_t*>(wsm_raw);   // [2 maps][64][pq]
  bf16_t* Ks = Qs + 2 * kWmRows * pq;                // [2 buffers][2 maps][64][pq]
  bf16_t* Vs = Ks + 4 * kWmKeys * pq;                // [2 buffers][64][pv]
  const int32_t* it = a.items + blockIdx.x * 4;
  const int first_row = it[0], n_tok = it[1], slot = it[2], first_pos = it[3];
  const int kvh = blockIdx.y, rep = a.H / a.G, n_rows = n_tok * rep;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int qchunks = d >> 3, vchunks = dv >> 3;
  for (int i = tid; i < 2 * kWmRows * qchunks; i += blockDim.x) {
    const int mm = i / (kWmRows * qchunks), r2 = i - mm * kWmRows * qchunks, row = r2 / qchunks, c = r2 - row * qchunks;
    bf16_t* dst = Qs + (mm * kWmRows + row) * pq + c * 8;
    if (row < n_rows) w_cp_async16(wsmem_u32(dst), a.q + (long long)(first_row + row / rep) * a.ldq + ((kvh * rep + row % rep) * 2 + mm) * d + c * 8);
    else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
  }
  const int row0 = warp * 16 + g, row1 = row0 + 8;
  const int p0 = row0 < n_rows ? first_pos + row0 / rep : -1, p1 = row1 < n_rows ? first_pos + row1 / rep : -1;   // -1: no such row
  const int h0 = kvh * rep + row0 % rep, h1 = kvh * rep + row1 % rep;
  const int32_t* bt = a.bt + (long long)slot * a.max_pages;
  int k_begin = max(0, first_pos - a.window + 1);
  const int k_end = first_pos + n_tok;
  int kept_end = min(a.keep_first, k_begin);
  if (kept_end == k_begin) k_begin = 0, kept_end = 0;
  const int kept_tiles = (kept_end + kWmKeys - 1) / kWmKeys, n_tiles = kept_tiles + (k_end - k_begin + kWmKeys - 1) / kWmKeys;
  const int roww = a.G * (2 * d + dv);
  auto stage = [&](int buf, int tile) {
    const int j0 = tile < kept_tiles ? tile * kWmKeys : k_begin + (tile - kept_tiles) * kWmKeys, j_end = tile < kept_tiles ? kept_end : k_end;
    const int key = tid >> 1, half = tid & 1, j = j0 + key;
    bf16_t* k0d = Ks + ((buf * 2 + 0) * kWmKeys + key) * pq;
    bf16_t* k1d = Ks + ((buf * 2 + 1) * kWmKeys + key) * pq;
    bf16_t* vd = Vs + (buf * kWmKeys + key) * pv;
    if (j < j_end) {
      const bf16_t* row = a.pool + ((long long)bt[j / a.page_size] * a.page_size + j % a.page_size) * roww;
      const bf16_t* ks = row + kvh * 2 * d;            // the two maps' keys of this key/value head lie side by side
      const bf16_t* vs = row + a.G * 2 * d + kvh * dv;
      for (int c = half; c < qchunks; c += 2) {
        w_cp_async16(wsmem_u32(k0d + c * 8), ks + c * 8);
        w_cp_async16(wsmem_u32(k1d + c * 8), ks + d + c * 8);
      }
      for (int c = half; c < vchunks; c += 2) w_cp_async16(wsmem_u32(vd + c * 8), vs + c * 8);
    } else {
      for (int c = half; c < qchunks; c += 2) {
        *reinterpret_cast<uint4*>(k0d + c * 8) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(k1d + c * 8) = make_uint4(0, 0, 0, 0);
      }
      for (int c = half; c < vchunks; c += 2) *reinterpret_cast<uint4*>(vd + c * 8) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float m0[2] = {-INFINITY, -INFINITY}, m1[2] = {-INFINITY, -INFINITY}, l0[2] = {0.f, 0.f}, l1[2] = {0.f, 0.f};
  float o[2][NV][4];
#pragma unroll
  for (int mm = 0; mm < 2; ++mm)
#pragma unroll
    for (int j = 0; j < NV; ++j) o[mm][j][0] = o[mm][j][1] = o[mm][j][2] = o[mm][j][3] = 0.f;
  const int nv = dv >> 3;
  constexpr float kLog2e = 1.4426950408889634f;
  const float sc2 = a.scale * kLog2e;   // scores in base-2 units
  stage(0, 0);
  for (int kt = 0; kt < n_tiles; ++kt) {
    const int buf = kt & 1;
    const int j0 = kt < kept_tiles ? kt * kWmKeys : k_begin + (kt - kept_tiles) * kWmKeys, j_end = kt < kept_tiles ? kept_end : k_end;
    if (kt + 1 < n_tiles) {
      stage(buf ^ 1, kt + 1);   // released by the barrier that ended the previous tile
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (warp * 16 < n_rows) {
      const bf16_t* Vc = Vs + buf * kWmKeys * pv;
      const uint32_t v_base = wsmem_u32(Vc + ((lane & 7) + 8 * ((lane >> 3) & 1)) * pv + 8 * (lane >> 4));
#pragma unroll
      for (int mm = 0; mm < 2; ++mm) {
        const bf16_t* Kc = Ks + (buf * 2 + mm) * kWmKeys * pq;
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        const uint32_t q_base = wsmem_u32(Qs + (mm * kWmRows + warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * pq + 8 * (lane >> 4));
        const uint32_t k_base = wsmem_u32(Kc + ((lane & 7) + 8 * (lane >> 4)) * pq + 8 * ((lane >> 3) & 1));
        for (int kk = 0; kk < d; kk += 16) {
          uint32_t a0, a1, a2, a3;
          w_ldsm_x4(q_base + kk * 2, a0, a1, a2, a3);
#pragma unroll
          for (int n2 = 0; n2 < 4; ++n2) {
            uint32_t b0, b1, b2, b3;
            w_ldsm_x4(k_base + (n2 * 16 * pq + kk) * 2, b0, b1, b2, b3);
            w_mma_bf16(s[2 * n2], a0, a1, a2, a3, b0, b1);
            w_mma_bf16(s[2 * n2 + 1], a0, a1, a2, a3, b2, b3);
          }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = j0 + n * 8 + 2 * t4 + (e & 1);
            const int dist = (e < 2 ? p0 : p1) - key;
            s[n][e] = (key < j_end && dist >= 0 && (dist < a.window || key < a.keep_first)) ? s[n][e] * sc2 : -INFINITY;
          }
          mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
          mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0[mm], mx0), mn1 = fmaxf(m1[mm], mx1);
        const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;   // rows that see nothing yet
        const float c0 = exp2f(m0[mm] - ms0), c1 = exp2f(m1[mm] - ms1);
        m0[mm] = mn0;
        m1[mm] = mn1;
        float rs0 = 0.f, rs1 = 0.f;
        uint32_t p[8][2];
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          p[n][0] = w_pack2(exp2f(s[n][0] - ms0), exp2f(s[n][1] - ms0));
          p[n][1] = w_pack2(exp2f(s[n][2] - ms1), exp2f(s[n][3] - ms1));
          // the denominator sums the ROUNDED probabilities, the ones the numerator uses
          const float2 f0 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&p[n][0]));
          const float2 f1 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&p[n][1]));
          rs0 += f0.x + f0.y;
          rs1 += f1.x + f1.y;
        }
        l0[mm] = l0[mm] * c0 + rs0;
        l1[mm] = l1[mm] * c1 + rs1;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          o[mm][j][0] *= c0;
          o[mm][j][1] *= c0;
          o[mm][j][2] *= c1;
          o[mm][j][3] *= c1;
        }
#pragma unroll
        for (int kb16 = 0; kb16 < 4; ++kb16) {
          const uint32_t a0 = p[2 * kb16][0], a1 = p[2 * kb16][1], a2 = p[2 * kb16 + 1][0], a3 = p[2 * kb16 + 1][1];
#pragma unroll
          for (int j = 0; j < NV; j += 2) {
            if (j < nv) {   // dv is a multiple of 16: tiles come in pairs
              uint32_t b0, b1, b2, b3;
              w_ldsm_x4_t(v_base + (kb16 * 16 * pv + j * 8) * 2, b0, b1, b2, b3);
              w_mma_bf16(o[mm][j], a0, a1, a2, a3, b0, b1);
              w_mma_bf16(o[mm][j + 1], a0, a1, a2, a3, b2, b3);
            }
          }
        }
      }
    }
    __syncthreads();   // every warp is done with this tile's buffers
  }
  float i0[2], i1[2];
#pragma unroll
  for (int mm = 0; mm < 2; ++mm) {
    float x = l0[mm], y = l1[mm];
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    x += __shfl_xor_sync(0xffffffffu, x, 2);
    y += __shfl_xor_sync(0xffffffffu, y, 1);
    y += __shfl_xor_sync(0xffffffffu, y, 2);
    i0[mm] = 1.f / x;
    i1[mm] = 1.f / y;
  }
  // o = a1 - lambda a2 in place of the first map's accumulators; a row's dv values are spread over the four lanes of its quad
  float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    if (j < nv) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float v = e < 2 ? o[0][j][e] * i0[0] - a.lambda * (o[1][j][e] * i0[1]) : o[0][j][e] * i1[0] - a.lambda * (o[1][j][e] * i1[1]);
        o[0][j][e] = v;
        if (e < 2) ss0 = fmaf(v, v, ss0);
        else ss1 = fmaf(v, v, ss1);
      }
    }
  }
  ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1);
  ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
  ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1);
  ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
  const float f0 = a.mult / sqrtf(ss0 / (float)dv + a.eps), f1 = a.mult / sqrtf(ss1 / (float)dv + a.eps);
  const long long t0 = first_row + row0 / rep, t1 = first_row + row1 / rep;
  TO* out0 = static_cast<TO*>(a.out) + t0 * a.ldo + h0 * dv;
  TO* out1 = static_cast<TO*>(a.out) + t1 * a.ldo + h1 * dv;
  auto act = [&](float z) { return a.gate_act == 2 ? 1.f / (1.f + __expf(-z)) : (a.gate_act == 1 ? z / (1.f + __expf(-z)) : z); };
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    if (j < nv) {
      const int col = j * 8 + 2 * t4;
      if (row0 < n_rows) {
        float g0 = 1.f, g1 = 1.f;
        if (a.gate != nullptr) {
          const float2 z = *reinterpret_cast<const float2*>(a.gate + t0 * a.ldg + h0 * dv + col);
          g0 = act(z.x), g1 = act(z.y);
        }
        w_st_pair(out0 + col, o[0][j][0] * f0 * g0, o[0][j][1] * f0 * g1);
      }
      if (row1 < n_rows) {
        float g0 = 1.f, g1 = 1.f;
        if (a.gate != nullptr) {
          const float2 z = *reinterpret_cast<const float2*>(a.gate + t1 * a.ldg + h1 * dv + col);
          g0 = act(z.x), g1 = act(z.y);
        }
        w_st_pair(out1 + col, o[0][j][2] * f1 * g0, o[0][j][3] * f1 * g1);
      }
    }
  }
}

// Two score maps of a head -> one output: o = a1 - lambda a2, o / sqrt(mean(o^2) + eps) over the head's dv values, times a constant,
// times an elementwise gate. One CTA per row, a warp per head.
template <typename TY>
__global__ void __launch_bounds__(256) diff_heads_gate_kernel(const float* __restrict__ a, long long lda, int H, int dv, float lambda,
                                                              float mult, float eps, const float* __restrict__ gate, long long ldg,
                                                              int gate_act, TY* __restrict__ y, long long ldy) {
  const long long t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int h = warp; h < H; h += nw) {
    const float* a1 = a + t * lda + (long long)2 * h * dv;
    const float* a2 = a1 + dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) {
      const float o = a1[c] - lambda * a2[c];
      ss = fmaf(o, o, ss);
    }
    ss = seq_warp_sum(ss);
    const float f = mult / sqrtf(ss / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) {
      float o = (a1[c] - lambda * a2[c]) * f;
      if (gate != nullptr) {
        const float z = gate[t * ldg + h * dv + c];
        o *= gate_act == 2 ? 1.f / (1.f + expf(-z)) : (gate_act == 1 ? z / (1.f + expf(-z)) : z);
      }
      stf(y + t * ldy + h * dv + c, o);
    }
  }
}

}  // namespace omc

using namespace omc;

extern "C" int omc_diff_heads_gate(const float* a, long long lda, int T, int H, int dv, float lambda, float mult, float eps,
                                   const float* gate, long long ldg, int gate_act, void* y, int y_dt, long long ldy, void* stream) {
  if (a == nullptr || y == nullptr || T < 0 || H <= 0 || dv <= 0 || gate_act < 0 || gate_act > 2)
    return set_error(OMC_ERR_ARG, "omc_diff_heads_gate: bad argument");
  if (T == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(y_dt, TY, {
    diff_heads_gate_kernel<TY><<<T, 256, 0, st>>>(a, lda, H, dv, lambda, mult, eps, gate, ldg, gate_act, static_cast<TY*>(y), ldy);
  })
  return check_launch("omc_diff_heads_gate");
}

extern "C" int omc_qk_norm_kv_store(const float* q, long long ldq, int nq, int q_group, const void* wq, const float* k, long long ldk, int nk,
                                    int k_group, const void* wk, int w_dt, const float* v, long long ldv, int nv, float eps, int T,
                                    const int32_t* pos, const int32_t* slot, const int32_t* block_table, int max_pages, int page_size,
                                    void* pool, void* q_out, long long ldqo, int dt, void* stream) {
  if (q == nullptr || wq == nullptr || k == nullptr || wk == nullptr || v == nullptr || pos == nullptr || slot == nullptr ||
      block_table == nullptr || pool == nullptr || q_out == nullptr || T < 0 || nq <= 0 || nk <= 0 || nv <= 0 || page_size <= 0 || max_pages <= 0 ||
      q_group < 0 || k_group < 0 || (q_group > 0 && nq % q_group) || (k_group > 0 && nk % k_group))
    return set_error(OMC_ERR_ARG, "omc_qk_norm_kv_store: bad argument");
  if (T == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(w_dt, TW, OMC_DT_SWITCH(dt, TC, {
    qk_norm_kv_store_kernel<TW, TC><<<T, 256, 0, st>>>(q, ldq, nq, q_group, static_cast<const TW*>(wq), k, ldk, nk, k_group, static_cast<const TW*>(wk), v,
                                                       ldv, nv, eps, pos, slot, block_table, max_pages, page_size,
                                                       static_cast<TC*>(pool), static_cast<TC*>(q_out), ldqo);
  }))
  return check_launch("omc_qk_norm_kv_store");
}

extern "C" int omc_window_attn(const void* q, long long ldq, int T, int H, int G, int d, int dv, int maps, const void* pool, int dt,
                               const int32_t* block_table, int max_pages, int page_size, const int32_t* pos, const int32_t* slot,
                               int window, int keep_first, float scale, float softcap, const float* dist_bias, const float* sink,
                               const float* gate, long long ldg, int gate_act, void* out, int out_dt, long long ldo, void* stream) {
  if (q == nullptr || pool == nullptr || block_table == nullptr || pos == nullptr || slot == nullptr || out == nullptr || T < 0 ||
      H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || maps < 1 || window < 1 || keep_first < 0 || page_size <= 0 || max_pages <= 0 ||
      gate_act < 0 || gate_act > 2)
    return set_error(OMC_ERR_ARG, "omc_window_attn: bad argument");
  if (T == 0) return OMC_OK;
  if (dv > 32 * kWinMaxPerLane) return set_error(OMC_ERR_SHAPE, "omc_window_attn: value width above 256");
  if ((long long)H * maps > 65535) return set_error(OMC_ERR_SHAPE, "omc_window_attn: more than 65535 heads");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = sizeof(float) * ((size_t)d + (size_t)kWinWarps * dv + 2 * kWinWarps);
  if (smem > 48 * 1024) return set_error(OMC_ERR_SHAPE, "omc_window_attn: head width too large");
  OMC_DT_SWITCH(dt, TC, OMC_DT_SWITCH(out_dt, TY, {
    window_attn_kernel<TC, TC, TY><<<dim3(T, H * maps), kWinWarps * 32, smem, st>>>(static_cast<const TC*>(q), ldq, H, G, d, dv, maps,
                                                                                   static_cast<const TC*>(pool), block_table, max_pages,
                                                                                   page_size, pos, slot, window, keep_first, scale, softcap,
                                                                                   dist_bias, sink, gate, ldg, gate_act, static_cast<TY*>(out), ldo);
  }))
  return check_launch("omc_window_attn");
}

extern "C" int omc_window_attn_mma_ok(int H, int G, int d, int dv) {
  if (H <= 0 || G <= 0 || H % G) return 0;
  const int rep = H / G;
  return (d % 16 == 0 && dv % 16 == 0 && d >= 16 && d <= 256 && dv >= 16 && dv <= 128 && rep <= 64 && 64 % rep == 0) ? 1 : 0;
}

extern "C" int omc_window_attn_mma(const void* q, long long ldq, int T, int H, int G, int d, int dv, int maps, const void* pool,
                                   const int32_t* block_table, int max_pages, int page_size, const int32_t* items, int n_items,
                                   const int32_t* pos, const int32_t* slot, int window, int keep_first, float scale, float softcap,
                                   const float* dist_bias, const float* sink, const float* gate, long long ldg, int gate_act, void* out,
                                   int out_dt, long long ldo, void* stream) {
  if (q == nullptr || pool == nullptr || block_table == nullptr || out == nullptr || T < 0 || window < 1 || maps < 1 || keep_first < 0 || page_size <= 0 ||
      gate_act < 0 || gate_act > 2 || max_pages <= 0 || (items == nullptr && (pos == nullptr || slot == nullptr)) || n_items < 0)
    return set_error(OMC_ERR_ARG, "omc_window_attn_mma: bad argument");
  if (!omc_window_attn_mma_ok(H, G, d, dv) || ldq % 8 || ldo % 2 || reinterpret_cast<uintptr_t>(q) % 16 || reinterpret_cast<uintptr_t>(pool) % 16)
    return set_error(OMC_ERR_SHAPE, "omc_window_attn_mma: shape or alignment not supported (see omc_window_attn_mma_ok)");
  const int n = items != nullptr ? n_items : T;
  if (n == 0) return OMC_OK;
  if ((long long)G * maps > 65535) return set_error(OMC_ERR_SHAPE, "omc_window_attn_mma: more than 65535 key/value heads");
  WinMmaArgs a{static_cast<const bf16_t*>(q), ldq, static_cast<const bf16_t*>(pool), block_table, items, pos, slot, dist_bias, sink, gate, ldg,
               gate_act, out, ldo, max_pages, page_size, H, G, d, dv, window, maps, keep_first, scale, softcap, kWmRows, 0};
  if (items == nullptr) a.q_rows = ((H / G + 15) / 16) * 16;   // one token per item: only H / G rows exist, and a smaller tile lets more CTAs share an SM
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  size_t smem = sizeof(bf16_t) * ((size_t)a.q_rows * (d + 8) + 2 * (size_t)kWmKeys * (d + 8) + 2 * (size_t)kWmKeys * (dv + 8));
  const size_t bias_bytes = sizeof(float) * (size_t)window * (H / G);
  if (dist_bias != nullptr && bias_bytes <= 64 * 1024) {
    a.bias_in_smem = 1;
    smem += bias_bytes;
  }
  dim3 grid(n, G * maps);
  // one token per item and at most 16 rows: one warp computes, a second helps staging - half the registers per CTA, so that
  // (with the smaller query tile) four CTAs share an SM instead of three
  const int threads = a.q_rows == 16 ? 64 : 128;
#define OMC_WIN_LAUNCH(NV, TO)                                                                                      \
  do {                                                                                                              \
    static bool attr_done[kMaxDevices] = {};                                                                        \
    if (!attr_done[cur_device()]) {                                                                                 \
      cudaFuncSetAttribute(window_attn_mma_kernel<NV, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
      attr_done[cur_device()] = true;                                                                               \
    }                                                                                                               \
    window_attn_mma_kernel<NV, TO><<<grid, threads, smem, st>>>(a);                                                     \
  } while (0)
  if (out_dt == OMC_DT_BF16) {
    if (dv <= 64) OMC_WIN_LAUNCH(8, bf16_t);
    else OMC_WIN_LAUNCH(16, bf16_t);
  } else if (out_dt == OMC_DT_F32) {
    if (dv <= 64) OMC_WIN_LAUNCH(8, float);
    else OMC_WIN_LAUNCH(16, float);
  } else {
    return set_error(OMC_ERR_ARG, "omc_window_attn_mma: unknown output dtype");
  }
#undef OMC_WIN_LAUNCH
  return check_launch("omc_window_attn_mma");
}

static size_t diff_pair_smem(int d, int dv) {
  return sizeof(bf16_t) * (2 * (size_t)kWmRows * (d + 8) + 4 * (size_t)kWmKeys * (d + 8) + 2 * (size_t)kWmKeys * (dv + 8));
}

extern "C" int omc_diff_attn_pair_ok(int H, int G, int d, int dv) {
  return (omc_window_attn_mma_ok(H, G, d, dv) && diff_pair_smem(d, dv) <= 200 * 1024) ? 1 : 0;
}

extern "C" int omc_diff_attn_pair(const void* q, long long ldq, int T, int H, int G, int d, int dv, const void* pool,
                                  const int32_t* block_table, int max_pages, int page_size, const int32_t* items, int n_items, int window,
                                  int keep_first, float scale, float lambda, float mult, float eps, const float* gate, long long ldg,
                                  int gate_act, void* out, int out_dt, long long ldo, void* stream) {
  if (q == nullptr || pool == nullptr || block_table == nullptr || items == nullptr || out == nullptr || T < 0 || n_items < 0 || window < 1 ||
      keep_first < 0 || page_size <= 0 || max_pages <= 0 || gate_act < 0 || gate_act > 2)
    return set_error(OMC_ERR_ARG, "omc_diff_attn_pair: bad argument");
  if (!omc_diff_attn_pair_ok(H, G, d, dv) || ldq % 8 || ldo % 2 || ldg % 2 || reinterpret_cast<uintptr_t>(q) % 16 ||
      reinterpret_cast<uintptr_t>(pool) % 16 || reinterpret_cast<uintptr_t>(gate) % 8)
    return set_error(OMC_ERR_SHAPE, "omc_diff_attn_pair: shape or alignment not supported (see omc_diff_attn_pair_ok)");
  if (n_items == 0) return OMC_OK;
  if (G > 65535) return set_error(OMC_ERR_SHAPE, "omc_diff_attn_pair: more than 65535 key/value heads");
  DiffPairArgs a{static_cast<const bf16_t*>(q), ldq, static_cast<const bf16_t*>(pool), block_table, items, gate, ldg, out, ldo,
                 max_pages, page_size, H, G, d, dv, window, keep_first, gate_act, scale, lambda, mult, eps};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = diff_pair_smem(d, dv);
  dim3 grid(n_items, G);
#define OMC_PAIR_LAUNCH(NV, TO)                                                                                    \
  do {                                                                                                             \
    static bool attr_done[kMaxDevices] = {};                                                                       \
    if (!attr_done[cur_device()]) {                                                                                \
      cudaFuncSetAttribute(diff_attn_pair_kernel<NV, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
      attr_done[cur_device()] = true;                                                                              \
    }                                                                                                              \
    diff_attn_pair_kernel<NV, TO><<<grid, 128, smem, st>>>(a);                                                     \
  } while (0)
  if (out_dt == OMC_DT_BF16) {
    if (dv <= 64) OMC_PAIR_LAUNCH(8, bf16_t);
    else OMC_PAIR_LAUNCH(16, bf16_t);
  } else if (out_dt == OMC_DT_F32) {
    if (dv <= 64) OMC_PAIR_LAUNCH(8, float);
    else OMC_PAIR_LAUNCH(16, float);
  } else {
    return set_error(OMC_ERR_ARG, "omc_diff_attn_pair: unknown output dtype");
  }
#undef OMC_PAIR_LAUNCH
  return check_launch("omc_diff_attn_pair");
}

extern "C" int omc_pos_qkv_store(const float* q, long long ldq, int H, const float* k, long long ldk, int G, int d, const float* v, long long ldv,
                                 int dv, const float* freq, int rot_dims, float temp_coef, int temp_every, int v_unit, float eps, int T,
                                 const int32_t* pos, const int32_t* slot, const int32_t* block_table, int max_pages, int page_size, void* pool,
                                 void* q_out, long long ldqo, int dt, void* stream) {
  if (q == nullptr || k == nullptr || v == nullptr || pos == nullptr || slot == nullptr || block_table == nullptr || pool == nullptr ||
      q_out == nullptr || T < 0 || H <= 0 || G <= 0 || d <= 0 || dv <= 0 || page_size <= 0 || max_pages <= 0 ||
      (freq != nullptr && (rot_dims < 0 || rot_dims > d || rot_dims % 2)) || (temp_coef != 0.f && temp_every <= 0))
    return set_error(OMC_ERR_ARG, "omc_pos_qkv_store: bad argument");
  if (T == 0) return OMC_OK;
  const size_t smem = freq != nullptr ? sizeof(float) * (size_t)rot_dims : 0;
  if (smem > 48 * 1024) return set_error(OMC_ERR_SHAPE, "omc_pos_qkv_store: more than 12288 rotated dimensions");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(dt, TC, {
    pos_qkv_store_kernel<TC><<<T, 256, smem, st>>>(q, ldq, H, k, ldk, G, d, v, ldv, dv, freq, rot_dims, temp_coef, temp_every, v_unit, eps, pos,
                                                   slot, block_table, max_pages, page_size, static_cast<TC*>(pool), static_cast<TC*>(q_out), ldqo);
  })
  return check_launch("omc_pos_qkv_store");
}
