// Mixers that carry a fixed-size state per sequence instead of a growing cache: a short causal convolution per channel whose
// last inputs are state, and the family of linear-state recurrences
//     S <- diag(g_t) S;   u_t = beta_t (v_t - S^T k_t)  (delta rule)  or  u_t = v_t  (plain outer-product sum);
//     S <- S + k_t u_t^T;   o_t = S^T q_t
// with the decay g_t constant per head, one per token and head, or one per token, head and key channel, and the gated RMS norm
// that follows them. Rows of a step are addressed by (slot, position); the rows of one request are consecutive and ascending.
// A portion that starts at position 0 starts from a zero state, so a slot needs no clearing when it is handed to a new request.
// Everything here is fp32: state, decays and their logarithms, softplus / exponentials, step sizes, unit norms.
//
// The recurrence is evaluated token by token in every case - prompt portions and single decoded tokens run the same
// instructions in the same order, which makes the result independent of how a prompt is cut. Its parallelism is over the
// independent COLUMNS of S: column j of a head's state only ever meets v[:, j], so a CTA owns 32 columns of one head of one
// portion; a thread holds an eighth of the state elements of TWO neighbouring columns as packed fp32 pairs (one fma.rn.f32x2 serves
// both columns, and a key or query value read from shared memory is used twice), and the eight lanes of a column pair finish the
// two dot products of a token with three shuffles each. Tokens are staged 16 at a time in shared memory by cp.async, one chunk ahead of the one being
// computed (decays, sigmoid and silu applied in place on arrival), so the sequential loop touches registers and shared memory only.
#include "seq_common.cuh"

namespace omc {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
// sigmoid(z)^p - 1 = expm1(p * log sigmoid(z)), log sigmoid(z) = -softplus(-z). The decay is kept as its distance from 1: rounded to
// fp32 itself, a decay close to 1 loses most of the digits of 1 - decay, and the state multiplies by it once per token.
__device__ __forceinline__ float sigmoid_pow_m1_f(float z, float p) { return expm1f(-p * softplus_f(-z)); }

// ---- causal convolution (+ silu) (+ unit vectors) ---------------------------------------------------------------------------
// One CTA per (1 or 8 consecutive rows, block of channels; blocks are whole unit-vector groups). Tap j of `taps` multiplies the input
// `taps - 1 - j` positions back: an earlier row of the same step when that row belongs to the same request, else the state ring
// state[slot][position % (taps - 1)][channel], else (before position 0) zero. save_here: every row of the step is a request of
// its own, so the row's input goes into its ring from this kernel, after the reads (no other CTA reads that ring).
constexpr int kConvRows = 8;    // rows per CTA of a long step: neighbouring rows read each other's inputs, which then come from L1
constexpr int kConvMaxTaps = 32;

template <typename TW, typename TY>
__global__ void __launch_bounds__(256) causal_conv_silu_kernel(const float* __restrict__ x, long long ldx, int T, int ch, int ch_block,
                                                               int rows_per_cta, const TW* __restrict__ w, const TW* __restrict__ bias, int taps,
                                                               const int32_t* __restrict__ pos, const int32_t* __restrict__ slot,
                                                               float* __restrict__ state, TY* __restrict__ y, long long ldy,
                                                               int unit_channels, int unit_group, float unit_eps, int scaled_channels,
                                                               float unit_mult, int save_here, int act) {
  extern __shared__ float tile[];  // [rows_per_cta][ch_block]
  __shared__ const float* src[kConvRows][kConvMaxTaps];   // where tap j of row r reads: a row of x, a ring entry, or nothing
  const int t0 = blockIdx.x * rows_per_cta, nr = min(rows_per_cta, T - t0);
  const int c0 = blockIdx.y * ch_block, nc = min(ch_block, ch - c0);
  const int R = taps - 1;
  if (threadIdx.x < nr * taps) {
    const int r = threadIdx.x / taps, j = threadIdx.x - r * taps;
    const int t = t0 + r, p = pos[t], s = slot[t], back = R - j, sp = p - back;
    const float* q = nullptr;
    if (sp >= 0) q = (back == 0 || (t - back >= 0 && slot[t - back] == s)) ? x + (long long)(t - back) * ldx : state + ((long long)s * R + sp % R) * ch;
    src[r][j] = q;
  }
  __syncthreads();
  for (int cl = threadIdx.x; cl < nc; cl += blockDim.x) {
    const int c = c0 + cl;
    const float b0 = bias != nullptr ? ldf(bias + c) : 0.f;
    for (int r = 0; r < nr; ++r) {
      float acc = b0;
#pragma unroll 4
      for (int j = 0; j < taps; ++j) {
        const float* q = src[r][j];
        const float xv = q != nullptr ? q[c] : 0.f;
        acc = fmaf(ldf(w + (long long)c * taps + j), xv, acc);
      }
      tile[r * ch_block + cl] = act ? silu_f(acc) : acc;
      // this thread is the only one that touches channel c of the ring: its write follows its reads
      if (save_here && R > 0) state[((long long)slot[t0 + r] * R + pos[t0 + r] % R) * ch + c] = x[(long long)(t0 + r) * ldx + c];
    }
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int unit_here = max(0, min(nc, unit_channels - c0));      // unit-vector channels of this block (whole groups)
  const int groups = unit_group > 0 ? unit_here / unit_group : 0;
  for (int rg = warp; rg < nr * groups; rg += nw) {
    const int r = rg / groups, g = rg - r * groups;
    float* row = tile + r * ch_block + g * unit_group;
    float ss = 0.f;
    for (int c = lane; c < unit_group; c += 32) ss = fmaf(row[c], row[c], ss);
    ss = seq_warp_sum(ss);
    const float f = (1.f / sqrtf(ss + unit_eps)) * (c0 + g * unit_group < scaled_channels ? unit_mult : 1.f);
    for (int c = lane; c < unit_group; c += 32) row[c] *= f;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < nr * nc; e += blockDim.x) {
    const int r = e / nc, cl = e - r * nc;
    stf(y + (long long)(t0 + r) * ldy + c0 + cl, tile[r * ch_block + cl]);
  }
}

// The same convolution (no activation) in front of an attention: the first nq + nk channels are queries and keys that get an RMS norm
// per `group` channels (a head, or one score map of a head) with the weights wq / wk [group]; queries go to q_out, normed keys and the
// remaining channels (values) to the row of (slot, position) in the paged cache [pages][page_size][ch - nq]. One launch instead of
// convolution, norm and append, and the convolved rows never travel through memory.
template <typename TW, typename TC>
__global__ void __launch_bounds__(256) conv_qk_norm_store_kernel(const float* __restrict__ x, long long ldx, int T, int ch, int ch_block,
                                                                 int rows_per_cta, const TW* __restrict__ w, int taps,
                                                                 const int32_t* __restrict__ pos, const int32_t* __restrict__ slot,
                                                                 float* __restrict__ state, int nq, int nk, int group,
                                                                 const TW* __restrict__ wq, const TW* __restrict__ wk, float eps,
                                                                 const int32_t* __restrict__ block_table, int max_pages, int page_size,
                                                                 TC* __restrict__ pool, TC* __restrict__ q_out, long long ldqo,
                                                                 int save_here) {
  extern __shared__ float tile[];  // [rows_per_cta][ch_block]
  __shared__ const float* src[kConvRows][kConvMaxTaps];
  __shared__ TC* dst_row[kConvRows];   // the cache row of every row of this CTA
  const int t0 = blockIdx.x * rows_per_cta, nr = min(rows_per_cta, T - t0);
  const int c0 = blockIdx.y * ch_block, nc = min(ch_block, ch - c0);
  const int R = taps - 1;
  if (threadIdx.x < nr * taps) {
    const int r = threadIdx.x / taps, j = threadIdx.x - r * taps;
    const int t = t0 + r, p = pos[t], s = slot[t], back = R - j, sp = p - back;
    const float* q = nullptr;
    if (sp >= 0) q = (back == 0 || (t - back >= 0 && slot[t - back] == s)) ? x + (long long)(t - back) * ldx : state + ((long long)s * R + sp % R) * ch;
    src[r][j] = q;
  }
  if (threadIdx.x >= 224 && threadIdx.x - 224 < nr) {
    const int r = threadIdx.x - 224, p = pos[t0 + r];
    const int page = block_table[(long long)slot[t0 + r] * max_pages + p / page_size];
    dst_row[r] = pool + ((long long)page * page_size + p % page_size) * (ch - nq);
  }
  __syncthreads();
  for (int cl = threadIdx.x; cl < nc; cl += blockDim.x) {
    const int c = c0 + cl;
    for (int r = 0; r < nr; ++r) {
      float acc = 0.f;
#pragma unroll 4
      for (int j = 0; j < taps; ++j) {
        const float* q = src[r][j];
        const float xv = q != nullptr ? q[c] : 0.f;
        acc = fmaf(ldf(w + (long long)c * taps + j), xv, acc);
      }
      tile[r * ch_block + cl] = acc;
      if (save_here && R > 0) state[((long long)slot[t0 + r] * R + pos[t0 + r] % R) * ch + c] = x[(long long)(t0 + r) * ldx + c];
    }
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int groups = max(0, min(nc, nq + nk - c0)) / group;      // normed groups of this block (blocks are whole groups)
  for (int rg = warp; rg < nr * groups; rg += nw) {
    const int r = rg / groups, g = rg - r * groups;
    float* row = tile + r * ch_block + g * group;
    const TW* wn = c0 + g * group < nq ? wq : wk;
    float ss = 0.f;
    for (int c = lane; c < group; c += 32) ss = fmaf(row[c], row[c], ss);
    ss = seq_warp_sum(ss);
    const float f = 1.f / sqrtf(ss / (float)group + eps);
    for (int c = lane; c < group; c += 32) row[c] = row[c] * f * ldf(wn + c);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < nr * nc; e += blockDim.x) {
    const int r = e / nc, cl = e - r * nc, c = c0 + cl;
    const float v = tile[r * ch_block + cl];
    if (c < nq) stf(q_out + (long long)(t0 + r) * ldqo + c, v);
    else stf(dst_row[r] + (c - nq), v);
  }
}

// The last taps - 1 inputs of every request of the step go into its ring (rows that are followed by taps - 1 more rows of the
// same request are not among them). A launch of its own when a request may have several rows: a row's ring entry is read by
// CTAs of other rows of the convolution kernel.
__global__ void __launch_bounds__(256) conv_state_save_kernel(const float* __restrict__ x, long long ldx, int ch, int R, int T,
                                                              const int32_t* __restrict__ pos, const int32_t* __restrict__ slot,
                                                              float* __restrict__ state) {
  const int t = blockIdx.x;
  const int s = slot[t];
  if (t + R < T && slot[t + R] == s) return;
  float* dst = state + ((long long)s * R + pos[t] % R) * ch;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < ch; c += gridDim.y * blockDim.x) dst[c] = x[(long long)t * ldx + c];
}

// ---- linear-state recurrence ----------------------------------------------------------------------------------------------
constexpr int kScanCols = 32, kScanLanes = 8, kScanTok = 16;

struct ScanArgs {
  const float* q;      // [T, ldq]: head g of kv_heads at columns g * dim
  const float* k;
  const float* v;      // [T, ldv]: head h at columns h * vdim
  long long ldq, ldk, ldv;
  int silu_in;         // q, k, v pass silu on the way in
  int decay_mode;      // 0: decay_const[h]; 1: a[t, h]; 2: a[t, h * dim + i]  (1, 2: g = exp(-exp(A_log[h]) softplus(a + dt_bias))); 3: g = a[t, h * dim + i];
                       // 4: g = sigmoid(a[t, h * dim + i] + dt_bias[h * dim + i])^decay_pow; 5: a[t, h * dim + i] holds g - 1
                       // (4 and 5 apply the decay as S + (g - 1) S)
  float decay_pow;     // mode 4
  float out_scale;     // o_t = out_scale * S^T q_t (a query scale, applied to the read-out)
  const float* decay_const;
  const float* a;
  long long lda;
  const float* A_log;    // fp32 [H]
  const float* dt_bias;  // fp32 [H] (mode 1) or [H * dim] (mode 2)
  const float* beta;     // raw [T, ldb]: beta = sigmoid; NULL: no delta correction (u = v)
  long long ldb;
  float* state;          // [slots][H][dim][vdim]
  float* out;            // [T, ldo]
  long long ldo;
  const int32_t* row_begin;  // [P + 1] first row of every portion
  const int32_t* pos;
  const int32_t* slot;
  int H, G, dim, vdim;
};

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src));
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src));
}

// Packed fp32 pairs (sm_100: one instruction, two IEEE fp32 operations): the recurrence's state lives in such pairs.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// Shared-memory place of key channel i: lane l = i / DPT owns DPT consecutive channels (read as float4), and a gap of four floats
// between the lanes' blocks moves them to different banks (the eight float4 reads of a quarter warp, at strides of 12, 20 or 36 floats, fall on different banks).
template <int DPT>
__device__ __forceinline__ int scan_place(int i) { return (i / DPT) * (DPT + 4) + (i % DPT); }

// Two stages of kScanTok tokens each: the raw inputs of the next chunk arrive by cp.async while the current chunk is computed;
// after arrival one pass turns them in place into what the recurrence uses (silu, decays, sigmoid). VEC: 16-byte copies
// (every row starts on a 16-byte boundary and the widths are multiples of four), else 4-byte copies.
template <int DPT, bool VEC>
__global__ void __launch_bounds__(kScanCols / 2 * kScanLanes) linear_state_scan_kernel(ScanArgs a) {
  extern __shared__ __align__(16) float sm[];
  constexpr int PITCH = kScanLanes * (DPT + 4);
  const int dim = a.dim;
  const bool chan = a.decay_mode >= 2;   // one decay per key channel: computed here (2, 4) or given (3, 5)
  const bool minus1 = a.decay_mode >= 4;  // the staged value is the decay minus one
  const int stage_floats = kScanTok * PITCH * (chan ? 3 : 2) + kScanTok * kScanCols + 2 * kScanTok;
  const int h = blockIdx.y, kvh = h / (a.H / a.G);
  const int col0 = blockIdx.x * kScanCols;
  const int r0 = a.row_begin[blockIdx.z], r1 = a.row_begin[blockIdx.z + 1];
  if (r1 <= r0) return;
  // thread = (lane over the key channels, PAIR of neighbouring columns): a packed register holds one key channel of both columns
  const int tid = threadIdx.x, lane = tid & (kScanLanes - 1), cp = tid / kScanLanes, col = col0 + 2 * cp;
  const bool ok0 = col < a.vdim, ok1 = col + 1 < a.vdim;
  for (int e = tid; e < 2 * stage_floats; e += blockDim.x) sm[e] = 0.f;   // the pads stay zero: they meet zero state only
  float* S = a.state + (((long long)a.slot[r0] * a.H + h) * dim) * a.vdim;
  f32x2 st[DPT];   // state elements (lane * DPT + r, col) and (lane * DPT + r, col + 1)
  const bool fresh = a.pos[r0] == 0;
#pragma unroll
  for (int r = 0; r < DPT; ++r) {
    const int i = lane * DPT + r;
    const bool ld = !fresh && i < dim;
    st[r] = pack2((ld && ok0) ? S[(long long)i * a.vdim + col] : 0.f, (ld && ok1) ? S[(long long)i * a.vdim + col + 1] : 0.f);
  }
  const float A = (a.decay_mode == 1 || a.decay_mode == 2) ? expf(a.A_log[h]) : 0.f;
  const float gconst = a.decay_mode == 0 ? a.decay_const[h] : 1.f;
  __syncthreads();

  auto issue = [&](int c0, int n, int stage) {
    float* sk = sm + stage * stage_floats;
    float* sq = sk + kScanTok * PITCH;
    float* sg = sq + kScanTok * PITCH;                       // [tok][PITCH] (per channel) or [tok]
    float* sv = sg + (chan ? kScanTok * PITCH : kScanTok);
    float* sb = sv + kScanTok * kScanCols;
    if (VEC) {
      const int d4 = dim >> 2;
      for (int e = tid; e < n * d4; e += blockDim.x) {
        const int tt = e / d4, i = (e - tt * d4) << 2, at = tt * PITCH + scan_place<DPT>(i);
        cp_async16(sk + at, a.k + (long long)(c0 + tt) * a.ldk + kvh * dim + i);
        cp_async16(sq + at, a.q + (long long)(c0 + tt) * a.ldq + kvh * dim + i);
        if (chan) cp_async16(sg + at, a.a + (long long)(c0 + tt) * a.lda + h * dim + i);
      }
      for (int e = tid; e < n * (kScanCols / 4); e += blockDim.x) {
        const int tt = e / (kScanCols / 4), j = (e - tt * (kScanCols / 4)) << 2;
        if (col0 + j < a.vdim) cp_async16(sv + tt * kScanCols + j, a.v + (long long)(c0 + tt) * a.ldv + h * a.vdim + col0 + j);
      }
    } else {
      for (int e = tid; e < n * dim; e += blockDim.x) {
        const int tt = e / dim, i = e - tt * dim, at = tt * PITCH + scan_place<DPT>(i);
        cp_async4(sk + at, a.k + (long long)(c0 + tt) * a.ldk + kvh * dim + i);
        cp_async4(sq + at, a.q + (long long)(c0 + tt) * a.ldq + kvh * dim + i);
        if (chan) cp_async4(sg + at, a.a + (long long)(c0 + tt) * a.lda + h * dim + i);
      }
      for (int e = tid; e < n * kScanCols; e += blockDim.x) {
        const int tt = e / kScanCols, j = e - tt * kScanCols;
        if (col0 + j < a.vdim) cp_async4(sv + e, a.v + (long long)(c0 + tt) * a.ldv + h * a.vdim + col0 + j);
      }
    }
    if (tid < n) {
      if (a.beta != nullptr) cp_async4(sb + tid, a.beta + (long long)(c0 + tid) * a.ldb + h);
      if (a.decay_mode == 1) cp_async4(sg + tid, a.a + (long long)(c0 + tid) * a.lda + h);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  issue(r0, min(kScanTok, r1 - r0), 0);
  int stage = 0;
  for (int c0 = r0; c0 < r1; c0 += kScanTok, stage ^= 1) {
    const int n = min(kScanTok, r1 - c0);
    if (c0 + kScanTok < r1) {
      issue(c0 + kScanTok, min(kScanTok, r1 - c0 - kScanTok), stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    float* sk = sm + stage * stage_floats;
    float* sq = sk + kScanTok * PITCH;
    float* sg = sq + kScanTok * PITCH;
    float* sv = sg + (chan ? kScanTok * PITCH : kScanTok);
    float* sb = sv + kScanTok * kScanCols;
    // raw inputs -> what the recurrence uses
    if (a.silu_in || a.decay_mode == 2 || a.decay_mode == 4) {
      for (int e = tid; e < n * dim; e += blockDim.x) {
        const int tt = e / dim, i = e - tt * dim, at = tt * PITCH + scan_place<DPT>(i);
        if (a.silu_in) {
          sk[at] = silu_f(sk[at]);
          sq[at] = silu_f(sq[at]);
        }
        if (a.decay_mode == 2) sg[at] = expf(-A * softplus_f(sg[at] + a.dt_bias[h * dim + i]));
        else if (a.decay_mode == 4) sg[at] = sigmoid_pow_m1_f(sg[at] + (a.dt_bias != nullptr ? a.dt_bias[h * dim + i] : 0.f), a.decay_pow);
      }
    }
    if (a.silu_in)
      for (int e = tid; e < n * kScanCols; e += blockDim.x) sv[e] = silu_f(sv[e]);
    if (tid < n) {
      sb[tid] = a.beta != nullptr ? sigmoid_f(sb[tid]) : 1.f;
      if (a.decay_mode == 1) sg[tid] = expf(-A * softplus_f(sg[tid] + a.dt_bias[h]));
      else if (a.decay_mode == 0) sg[tid] = gconst;
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float* kr = sk + tt * PITCH + lane * (DPT + 4);
      const float* qr = sq + tt * PITCH + lane * (DPT + 4);
      f32x2 da = 0ull, db = 0ull;   // (column, column + 1) partial dot products, two chains
      f32x2 k2[DPT];                // the key, each channel doubled: used again by the update
      const f32x2 gh = pack2(sg[chan ? 0 : tt], sg[chan ? 0 : tt]);
      const float* gr = sg + tt * PITCH + lane * (DPT + 4);
#pragma unroll
      for (int r = 0; r < DPT; r += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(kr + r);
        k2[r] = pack2(kv.x, kv.x), k2[r + 1] = pack2(kv.y, kv.y), k2[r + 2] = pack2(kv.z, kv.z), k2[r + 3] = pack2(kv.w, kv.w);
        if (chan) {
          const float4 gv = *reinterpret_cast<const float4*>(gr + r);
          if (minus1) {
            st[r] = fma2(st[r], pack2(gv.x, gv.x), st[r]), st[r + 1] = fma2(st[r + 1], pack2(gv.y, gv.y), st[r + 1]);
            st[r + 2] = fma2(st[r + 2], pack2(gv.z, gv.z), st[r + 2]), st[r + 3] = fma2(st[r + 3], pack2(gv.w, gv.w), st[r + 3]);
          } else {
            st[r] = mul2(st[r], pack2(gv.x, gv.x)), st[r + 1] = mul2(st[r + 1], pack2(gv.y, gv.y));
            st[r + 2] = mul2(st[r + 2], pack2(gv.z, gv.z)), st[r + 3] = mul2(st[r + 3], pack2(gv.w, gv.w));
          }
        } else {
          st[r] = mul2(st[r], gh), st[r + 1] = mul2(st[r + 1], gh), st[r + 2] = mul2(st[r + 2], gh), st[r + 3] = mul2(st[r + 3], gh);
        }
        da = fma2(st[r], k2[r], da), db = fma2(st[r + 1], k2[r + 1], db);
        da = fma2(st[r + 2], k2[r + 2], da), db = fma2(st[r + 3], k2[r + 3], db);
      }
      const float2 vv = *reinterpret_cast<const float2*>(sv + tt * kScanCols + 2 * cp);
      float u0 = vv.x, u1 = vv.y;
      if (a.beta != nullptr) {
        float a0, a1, b0, b1;
        unpack2(da, a0, a1);
        unpack2(db, b0, b1);
        float dot0 = a0 + b0, dot1 = a1 + b1;
#pragma unroll
        for (int m = 1; m < kScanLanes; m <<= 1) {
          dot0 += __shfl_xor_sync(0xffffffffu, dot0, m);
          dot1 += __shfl_xor_sync(0xffffffffu, dot1, m);
        }
        u0 = sb[tt] * (u0 - dot0);
        u1 = sb[tt] * (u1 - dot1);
      }
      const f32x2 u2 = pack2(u0, u1);
      f32x2 oa = 0ull, ob = 0ull;
#pragma unroll
      for (int r = 0; r < DPT; r += 4) {
        const float4 qv = *reinterpret_cast<const float4*>(qr + r);
        st[r] = fma2(k2[r], u2, st[r]), st[r + 1] = fma2(k2[r + 1], u2, st[r + 1]);
        st[r + 2] = fma2(k2[r + 2], u2, st[r + 2]), st[r + 3] = fma2(k2[r + 3], u2, st[r + 3]);
        oa = fma2(st[r], pack2(qv.x, qv.x), oa), ob = fma2(st[r + 1], pack2(qv.y, qv.y), ob);
        oa = fma2(st[r + 2], pack2(qv.z, qv.z), oa), ob = fma2(st[r + 3], pack2(qv.w, qv.w), ob);
      }
      float o0, o1, p0, p1;
      unpack2(oa, o0, o1);
      unpack2(ob, p0, p1);
      o0 += p0;
      o1 += p1;
#pragma unroll
      for (int m = 1; m < kScanLanes; m <<= 1) {
        o0 += __shfl_xor_sync(0xffffffffu, o0, m);
        o1 += __shfl_xor_sync(0xffffffffu, o1, m);
      }
      if (lane == 0) {
        float* dst = a.out + (long long)(c0 + tt) * a.ldo + h * a.vdim + col;
        if (ok0) dst[0] = o0 * a.out_scale;
        if (ok1) dst[1] = o1 * a.out_scale;
      }
    }
    __syncthreads();   // the next iteration's copies overwrite the stage that was just read
  }
#pragma unroll
  for (int r = 0; r < DPT; ++r) {
    const int i = lane * DPT + r;
    float lo, hi;
    unpack2(st[r], lo, hi);
    if (i < dim && ok0) S[(long long)i * a.vdim + col] = lo;
    if (i < dim && ok1) S[(long long)i * a.vdim + col + 1] = hi;
  }
}

// ---- elementwise preparation of a recurrence's inputs --------------------------------------------------------------------
// In place over x[t, :cols]: op 1: silu; op 2: x <- exp(-exp(A_log[c / group]) * softplus(x + bias[c])), the per-channel decay;
// op 3: x <- sigmoid(x + bias[c])^p - 1, the decay of a gated linear attention as its distance from 1.
// The recurrence can do both itself while it stages its inputs; for long portions one pass here is cheaper than doing it in
// every CTA that shares a head.
__global__ void __launch_bounds__(256) map_rows_kernel(float* __restrict__ x, long long ldx, int cols, long long total, int op,
                                                       const float* __restrict__ A_log, const float* __restrict__ bias, int group, float p_exp) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const long long t = e / cols;
  const int c = (int)(e - t * cols);
  float* p = x + t * ldx + c;
  if (op == 1) *p = silu_f(*p);
  else if (op == 3) *p = sigmoid_pow_m1_f(*p + (bias != nullptr ? bias[c] : 0.f), p_exp);
  else *p = expf(-expf(A_log[c / group]) * softplus_f(*p + bias[c]));
}

// ---- gated RMS norm over groups of a row ----------------------------------------------------------------------------------
// y[t, g * n + c] = x[t, g * n + c] / sqrt(mean_c x^2 + eps) * w[c] * act(gate[t, g * n + c]); a warp per group.
template <typename TW, typename TY>
__global__ void __launch_bounds__(256) gated_rms_kernel(const float* __restrict__ x, long long ldx, int groups, int n,
                                                        const TW* __restrict__ w, float eps, const float* __restrict__ gate,
                                                        long long ldg, int gate_act, TY* __restrict__ y, long long ldy) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const long long t = blockIdx.x;
  for (int g = blockIdx.y * nw + warp; g < groups; g += nw * gridDim.y) {
    const float* xr = x + t * ldx + (long long)g * n;
    float ss = 0.f;
    for (int c = lane; c < n; c += 32) ss = fmaf(xr[c], xr[c], ss);
    ss = seq_warp_sum(ss);
    const float rstd = 1.f / sqrtf(ss / (float)n + eps);
    for (int c = lane; c < n; c += 32) {
      float v = xr[c] * rstd * ldf(w + c);
      if (gate != nullptr) {
        const float z = gate[t * ldg + (long long)g * n + c];
        v *= gate_act == 1 ? silu_f(z) : (gate_act == 2 ? sigmoid_f(z) : z);
      }
      stf(y + t * ldy + (long long)g * n + c, v);
    }
  }
}


// ---- tanh norm + input convolution of a sublayer ----------------------------------------------------------------------------
// What a sublayer of a "tanh-norm" decoder reads: with the stream row x (optionally first updated by the previous sublayer's
// output, x <- x + a1 y1 + a2 y2), h = tanh(alpha x) * nw + nb (a norm without statistics) and u = h + sum_j cw[:, j] h_(t - taps + 1 + j),
// a causal convolution over time per channel whose last taps - 1 inputs h live in a ring per slot like the other convolutions'.
// A CTA owns (1 or 8 consecutive rows + the taps - 1 rows in front of them, a block of channels): h is evaluated once per tile
// element into shared memory, then every row's taps read the tile, a ring entry or nothing.
// tanh for the norm. FAST (bf16 output): 1 - 2 / (exp(2x) + 1) through the hardware exponential, absolute error of a few 1e-7 -
// far below the rounding of the output; otherwise the library function.
template <bool FAST>
__device__ __forceinline__ float tanh_norm_f(float x) {
  if (FAST) {
    const float e = exp2f(fminf(x, 20.f) * 2.8853900817779268f);
    return 1.f - __fdividef(2.f, e + 1.f);
  }
  return tanhf(x);
}
template <bool FAST, typename TW>
__device__ __forceinline__ float dyt_f(float x, float alpha, const TW* __restrict__ nw, const TW* __restrict__ nb, int c) {
  return fmaf(tanh_norm_f<FAST>(alpha * x), ldf(nw + c), ldf(nb + c));
}
template <typename T>
struct is_bf16_t { static constexpr bool value = false; };
template <>
struct is_bf16_t<bf16_t> { static constexpr bool value = true; };

constexpr int kDytRegTaps = 8;   // convolutions of up to this many taps keep a channel's weights in registers across the rows
constexpr int kDytRows = 8;      // rows per CTA of a long step: the taps - 1 halo rows in front are evaluated once more per CTA (16 rows were slower)

template <typename TW, typename TU>
__global__ void __launch_bounds__(256) dyt_conv_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ y1, long long ld1,
                                                       float a1, const float* __restrict__ y2, long long ld2, float a2,
                                                       float* __restrict__ x_out, long long ldxo, const float* __restrict__ alpha_p,
                                                       const TW* __restrict__ nw, const TW* __restrict__ nb, const TW* __restrict__ cw, int taps,
                                                       const int32_t* __restrict__ pos, const int32_t* __restrict__ slot,
                                                       float* __restrict__ state, TU* __restrict__ u, long long ldu, int T, int C, int ch_block,
                                                       int rows_per_cta, int save_here) {
  constexpr bool FAST = is_bf16_t<TU>::value;
  extern __shared__ float tile[];  // [rows_per_cta + taps - 1][ch_block]: h of the halo rows, then of the CTA's own rows
  // where tap j of row r reads: a row of the tile (src_tile >= 0), a ring entry (src_ring != NULL, indexed by the channel), or nothing
  __shared__ int src_tile[kDytRows][kConvMaxTaps];
  __shared__ const float* src_ring[kDytRows][kConvMaxTaps];
  const int R = taps - 1;
  const int t0 = blockIdx.x * rows_per_cta, nr = min(rows_per_cta, T - t0);
  const int c0 = blockIdx.y * ch_block, nc = min(ch_block, C - c0);
  const float alpha = *alpha_p;
  for (int e = threadIdx.x; e < nr * taps; e += blockDim.x) {
    const int r = e / taps, j = e - r * taps;
    const int t = t0 + r, p = pos[t], s = slot[t], back = R - j, sp = p - back;
    int ti = -1;
    const float* q = nullptr;
    if (sp >= 0) {
      if (back == 0 || (t - back >= 0 && slot[t - back] == s)) ti = R + r - back;
      else q = state + ((long long)s * R + sp % R) * C;
    }
    src_tile[r][j] = ti;
    src_ring[r][j] = q;
  }
  for (int cl = threadIdx.x; cl < nc; cl += blockDim.x) {
    const int c = c0 + cl;
    const float w_n = ldf(nw + c), b_n = ldf(nb + c);
#pragma unroll 4
    for (int i = 0; i < nr + R; ++i) {
      const int t = t0 - R + i;
      float h = 0.f;
      if (t >= 0) {
        float xv = x[(long long)t * ldx + c];
        if (y1 != nullptr) xv = fmaf(a1, y1[(long long)t * ld1 + c], xv);
        if (y2 != nullptr) xv = fmaf(a2, y2[(long long)t * ld2 + c], xv);
        if (i >= R && x_out != nullptr) x_out[(long long)t * ldxo + c] = xv;
        h = fmaf(tanh_norm_f<FAST>(alpha * xv), w_n, b_n);
      }
      tile[i * ch_block + cl] = h;
    }
  }
  __syncthreads();   // a thread reads its own channel only, but the pointer table came from other threads
  for (int cl = threadIdx.x; cl < nc; cl += blockDim.x) {
    const int c = c0 + cl;
    float wreg[kDytRegTaps];
    if (taps <= kDytRegTaps) {
#pragma unroll
      for (int j = 0; j < kDytRegTaps; ++j) wreg[j] = j < taps ? ldf(cw + (long long)c * taps + j) : 0.f;
    }
    for (int r = 0; r < nr; ++r) {
      const float h = tile[(R + r) * ch_block + cl];
      float acc = h;
      if (taps <= kDytRegTaps) {
#pragma unroll
        for (int j = 0; j < kDytRegTaps; ++j) {
          if (j < taps) {
            const int ti = src_tile[r][j];
            const float* q = src_ring[r][j];
            if (ti >= 0) acc = fmaf(wreg[j], tile[ti * ch_block + cl], acc);
            else if (q != nullptr) acc = fmaf(wreg[j], q[c], acc);
          }
        }
      } else {
        for (int j = 0; j < taps; ++j) {
          const int ti = src_tile[r][j];
          const float* q = src_ring[r][j];
          const float wj = ldf(cw + (long long)c * taps + j);
          if (ti >= 0) acc = fmaf(wj, tile[ti * ch_block + cl], acc);
          else if (q != nullptr) acc = fmaf(wj, q[c], acc);
        }
      }
      stf(u + (long long)(t0 + r) * ldu + c, acc);
      // every row is a request of its own: nobody else reads this ring, and this thread's reads of channel c came first
      if (save_here && R > 0) state[((long long)slot[t0 + r] * R + pos[t0 + r] % R) * C + c] = h;
    }
  }
}

// The ring update of a step whose requests may have several rows: h of the last taps - 1 rows of every request, recomputed from the
// (already updated) stream rows.
template <bool FAST, typename TW>
__global__ void __launch_bounds__(256) dyt_state_save_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ alpha_p,
                                                             const TW* __restrict__ nw, const TW* __restrict__ nb, int C, int R, int T,
                                                             const int32_t* __restrict__ pos, const int32_t* __restrict__ slot,
                                                             float* __restrict__ state) {
  const int t = blockIdx.x;
  const int s = slot[t];
  if (t + R < T && slot[t + R] == s) return;
  const float alpha = *alpha_p;
  float* dst = state + ((long long)s * R + pos[t] % R) * C;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) dst[c] = dyt_f<FAST>(x[(long long)t * ldx + c], alpha, nw, nb, c);
}

// ---- selective scan -------------------------------------------------------------------------------------------------------
// Per channel c a state S[c, :N] (fp32, in the request's slot):  S <- exp(dt_c A[c, :]) * S + dt_c x_c B_t;  y_c = S . C_t + D_c x_c,
// with dt = softplus(raw + bias) per channel and token, A = -exp(A_log), B_t / C_t shared by the channels; the output is gated,
// y * silu(z). Channels are independent: a CTA owns a block of channels of one request's portion, LANES neighbouring lanes share a
// channel (lane l holds the states l, l + LANES, ...), tokens go one after the other in chunks of kSelTok staged in shared memory.
// A portion whose first row has position 0 starts from S = 0.
constexpr int kSelTok = 16, kSelThreads = 128;

struct SelArgs {
  const void* x;
  long long ldx;
  const float* dt;
  long long lddt;
  const float* dt_bias;
  const float* B;
  long long ldb;
  const float* Cm;
  long long ldc;
  const float* A_log;
  const float* D;
  const float* z;
  long long ldz;
  float* state;
  void* y;
  long long ldy;
  const int32_t* row_begin;
  const int32_t* pos;
  const int32_t* slot;
  int inner, N;
};

// exp(x) - 1 for x <= 0 without losing the digits of a small x: a Taylor polynomial below 0.1 (truncation 1e-9 of x), the hardware
// exponential above, where its absolute error of ~1e-7 is small against the result and such a fast decay forgets within a few tokens.
__device__ __forceinline__ float expm1_decay_f(float x) {
  const float p = x * fmaf(x, fmaf(x, fmaf(x, fmaf(x, 1.f / 120.f, 1.f / 24.f), 1.f / 6.f), 0.5f), 1.f);
  const float e = exp2f(x * 1.4426950408889634f) - 1.f;
  return x > -0.1f ? p : e;
}

// LANES neighbouring lanes share a channel; lane l holds the states l, l + LANES, ... (P of them).
template <int LANES, int P, typename TD>
__global__ void __launch_bounds__(kSelThreads) selective_scan_kernel(SelArgs a) {
  constexpr int CH = kSelThreads / LANES;
  extern __shared__ float sm[];
  float* s_dt = sm;                          // [tok][CH]
  float* s_x = s_dt + kSelTok * CH;          // [tok][CH]
  float* s_y = s_x + kSelTok * CH;           // [tok][CH]
  float* s_B = s_y + kSelTok * CH;           // [tok][N]
  float* s_C = s_B + kSelTok * a.N;          // [tok][N]
  const int N = a.N, tid = threadIdx.x, lane = tid % LANES, cl = tid / LANES;
  const int c0 = blockIdx.x * CH, c = c0 + cl, ncl = min(CH, a.inner - c0);
  const bool live = c < a.inner;
  const int r0 = a.row_begin[blockIdx.y], r1 = a.row_begin[blockIdx.y + 1];
  if (r1 <= r0) return;
  const bool fresh = a.pos[r0] == 0;
  float* S = a.state + ((long long)a.slot[r0] * a.inner + (live ? c : 0)) * N;
  float st[P], A[P];
#pragma unroll
  for (int r = 0; r < P; ++r) {
    const int n = lane + r * LANES;
    const bool ok = live && n < N;
    st[r] = (ok && !fresh) ? S[n] : 0.f;
    A[r] = ok ? -expf(a.A_log[(long long)c * N + n]) : 0.f;
  }
  const float Dc = live ? a.D[c] : 0.f;
  const TD* xg = static_cast<const TD*>(a.x);
  TD* yg = static_cast<TD*>(a.y);
  for (int t0 = r0; t0 < r1; t0 += kSelTok) {
    const int n_tok = min(kSelTok, r1 - t0);
    for (int tt = tid / CH; tt < n_tok; tt += kSelThreads / CH) {
      const int j = tid % CH;
      if (j < ncl) {
        s_dt[tt * CH + j] = softplus_f(a.dt[(long long)(t0 + tt) * a.lddt + c0 + j] + a.dt_bias[c0 + j]);
        s_x[tt * CH + j] = ldf(xg + (long long)(t0 + tt) * a.ldx + c0 + j);
      }
    }
    for (int e = tid; e < n_tok * N; e += kSelThreads) {
      const int tt = e / N, n = e - tt * N;
      s_B[e] = a.B[(long long)(t0 + tt) * a.ldb + n];
      s_C[e] = a.Cm[(long long)(t0 + tt) * a.ldc + n];
    }
    __syncthreads();
    for (int tt = 0; tt < n_tok; ++tt) {
      const float dt = s_dt[tt * CH + cl], xv = s_x[tt * CH + cl], dx = dt * xv;
      const float* Bt = s_B + tt * N;
      const float* Ct = s_C + tt * N;
      float y = 0.f;
#pragma unroll
      for (int r = 0; r < P; ++r) {
        const int n = lane + r * LANES;
        if (n < N) {
          // the decay as S + (exp(dt A) - 1) S: a decay close to 1 would lose most of the digits of 1 - decay when rounded to
          // fp32 itself, and that error grows with every token the state remembers
          st[r] = fmaf(expm1_decay_f(dt * A[r]), st[r], st[r]) + dx * Bt[n];
          y = fmaf(st[r], Ct[n], y);
        }
      }
#pragma unroll
      for (int m = 1; m < LANES; m <<= 1) y += __shfl_xor_sync(0xffffffffu, y, m);
      if (lane == 0) s_y[tt * CH + cl] = fmaf(Dc, xv, y);
    }
    __syncthreads();
    for (int tt = tid / CH; tt < n_tok; tt += kSelThreads / CH) {
      const int j = tid % CH;
      if (j < ncl) {
        float y = s_y[tt * CH + j];
        if (a.z != nullptr) y *= silu_f(a.z[(long long)(t0 + tt) * a.ldz + c0 + j]);
        stf(yg + (long long)(t0 + tt) * a.ldy + c0 + j, y);
      }
    }
    // the next chunk's staging writes s_dt / s_x / s_B / s_C, which nobody reads any more; s_y is rewritten only after the next barrier
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < P; ++r) {
      const int n = lane + r * LANES;
      if (n < N) S[n] = st[r];
    }
  }
}

}  // namespace omc

using namespace omc;

extern "C" int omc_causal_conv(const float* x, long long ldx, int T, int ch, const void* w, const void* bias, int w_dt, int taps,
                               const int32_t* pos, const int32_t* slot, float* state, void* y, int y_dt, long long ldy, int act,
                               int unit_channels, int unit_group, float unit_eps, int scaled_channels, float unit_mult,
                               int single_rows, void* stream) {
  if (x == nullptr || w == nullptr || pos == nullptr || slot == nullptr || y == nullptr || T < 0 || ch <= 0 || taps < 1 || taps > kConvMaxTaps ||
      (taps > 1 && state == nullptr) || (act != OMC_CONV_LINEAR && act != OMC_CONV_SILU) || unit_channels < 0 || unit_channels > ch || (unit_channels > 0 && (unit_group <= 0 || unit_channels % unit_group)) ||
      (unit_channels > 0 && scaled_channels % unit_group))
    return set_error(OMC_ERR_ARG, "omc_causal_conv: bad argument");
  if (T == 0) return OMC_OK;
  // channel blocks of about 512 channels, whole unit-vector groups each
  int ch_block = 512;
  if (unit_channels > 0) ch_block = unit_group >= 512 ? unit_group : (512 / unit_group) * unit_group;
  if (ch_block > ch) ch_block = ch;
  if ((size_t)ch_block * kConvRows * sizeof(float) > 200 * 1024) return set_error(OMC_ERR_SHAPE, "omc_causal_conv: unit-vector group too wide for shared memory");
  const int blocks = (ch + ch_block - 1) / ch_block;
  if (blocks > 65535) return set_error(OMC_ERR_SHAPE, "omc_causal_conv: too many channel blocks");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rows_per_cta = T >= 256 ? kConvRows : 1;   // short steps (decode) keep one CTA per row: there are few rows to share anything
  const size_t smem = (size_t)ch_block * rows_per_cta * sizeof(float);
  OMC_DT_SWITCH(w_dt, TW, OMC_DT_SWITCH(y_dt, TY, {
    if (smem > 48 * 1024) cudaFuncSetAttribute(causal_conv_silu_kernel<TW, TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    causal_conv_silu_kernel<TW, TY><<<dim3((T + rows_per_cta - 1) / rows_per_cta, blocks), 256, smem, st>>>(
        x, ldx, T, ch, ch_block, rows_per_cta, static_cast<const TW*>(w), static_cast<const TW*>(bias), taps, pos, slot, state,
        static_cast<TY*>(y), ldy, unit_channels, unit_group, unit_eps, scaled_channels, unit_mult, single_rows ? 1 : 0, act == OMC_CONV_SILU ? 1 : 0);
  }))
  if (taps > 1 && !single_rows) conv_state_save_kernel<<<dim3(T, (ch + 1023) / 1024), 256, 0, st>>>(x, ldx, ch, taps - 1, T, pos, slot, state);
  return check_launch("omc_causal_conv");
}

extern "C" int omc_conv_qk_norm_kv_store(const float* x, long long ldx, int T, int ch, const void* w, int w_dt, int taps, const int32_t* pos,
                                         const int32_t* slot, float* state, int nq, int nk, int group, const void* wq, const void* wk,
                                         float eps, const int32_t* block_table, int max_pages, int page_size, void* pool, void* q_out,
                                         long long ldqo, int dt, int single_rows, void* stream) {
  if (x == nullptr || w == nullptr || pos == nullptr || slot == nullptr || wq == nullptr || wk == nullptr || block_table == nullptr ||
      pool == nullptr || q_out == nullptr || T < 0 || taps < 1 || taps > kConvMaxTaps || (taps > 1 && state == nullptr) || group <= 0 ||
      nq <= 0 || nk <= 0 || nq % group || nk % group || ch <= nq + nk || page_size <= 0 || max_pages <= 0)
    return set_error(OMC_ERR_ARG, "omc_conv_qk_norm_kv_store: bad argument");
  if (T == 0) return OMC_OK;
  int ch_block = group >= 512 ? group : (512 / group) * group;
  if (ch_block > ch) ch_block = ch;
  if ((size_t)ch_block * kConvRows * sizeof(float) > 200 * 1024) return set_error(OMC_ERR_SHAPE, "omc_conv_qk_norm_kv_store: group too wide for shared memory");
  const int blocks = (ch + ch_block - 1) / ch_block;
  if (blocks > 65535) return set_error(OMC_ERR_SHAPE, "omc_conv_qk_norm_kv_store: too many channel blocks");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rows_per_cta = T >= 256 ? kConvRows : 1;
  const size_t smem = (size_t)ch_block * rows_per_cta * sizeof(float);
  OMC_DT_SWITCH(w_dt, TW, OMC_DT_SWITCH(dt, TC, {
    if (smem > 48 * 1024) cudaFuncSetAttribute(conv_qk_norm_store_kernel<TW, TC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    conv_qk_norm_store_kernel<TW, TC><<<dim3((T + rows_per_cta - 1) / rows_per_cta, blocks), 256, smem, st>>>(
        x, ldx, T, ch, ch_block, rows_per_cta, static_cast<const TW*>(w), taps, pos, slot, state, nq, nk, group, static_cast<const TW*>(wq),
        static_cast<const TW*>(wk), eps, block_table, max_pages, page_size, static_cast<TC*>(pool), static_cast<TC*>(q_out), ldqo,
        single_rows ? 1 : 0);
  }))
  if (taps > 1 && !single_rows) conv_state_save_kernel<<<dim3(T, (ch + 1023) / 1024), 256, 0, st>>>(x, ldx, ch, taps - 1, T, pos, slot, state);
  return check_launch("omc_conv_qk_norm_kv_store");
}

extern "C" int omc_causal_conv_silu(const float* x, long long ldx, int T, int ch, const void* w, int w_dt, int taps,
                                    const int32_t* pos, const int32_t* slot, float* state, float* y, long long ldy,
                                    int unit_channels, int unit_group, float unit_eps, int scaled_channels, float unit_mult,
                                    int single_rows, void* stream) {
  return omc_causal_conv(x, ldx, T, ch, w, nullptr, w_dt, taps, pos, slot, state, y, OMC_DT_F32, ldy, OMC_CONV_SILU, unit_channels, unit_group,
                         unit_eps, scaled_channels, unit_mult, single_rows, stream);
}

extern "C" int omc_linear_state_scan(const float* q, long long ldq, const float* k, long long ldk, const float* v, long long ldv,
                                     int silu_in, int decay_mode, const float* decay_const, const float* a, long long lda,
                                     const float* A_log, const float* dt_bias, const float* beta, long long ldb, float* state,
                                     float* out, long long ldo, const int32_t* row_begin, int portions, const int32_t* pos,
                                     const int32_t* slot, int H, int G, int dim, int vdim, float decay_pow, float out_scale, void* stream) {
  if (q == nullptr || k == nullptr || v == nullptr || state == nullptr || out == nullptr || row_begin == nullptr || pos == nullptr ||
      slot == nullptr || portions < 0 || H <= 0 || G <= 0 || H % G || dim <= 0 || vdim <= 0 || decay_mode < 0 || decay_mode > 5 ||
      (decay_mode == 0 && decay_const == nullptr) || (decay_mode != 0 && a == nullptr) ||
      ((decay_mode == 1 || decay_mode == 2) && (A_log == nullptr || dt_bias == nullptr)))
    return set_error(OMC_ERR_ARG, "omc_linear_state_scan: bad argument");
  if (portions == 0) return OMC_OK;
  if (dim > 256) return set_error(OMC_ERR_SHAPE, "omc_linear_state_scan: key width above 256");
  if (portions > 65535 || H > 65535) return set_error(OMC_ERR_SHAPE, "omc_linear_state_scan: more than 65535 portions or heads");
  ScanArgs s{q, k, v, ldq, ldk, ldv, silu_in, decay_mode, decay_pow, out_scale, decay_const, a, lda, A_log, dt_bias, beta, ldb, state, out, ldo,
             row_begin, pos, slot, H, G, dim, vdim};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int dpt = dim <= 32 ? 4 : (dim <= 64 ? 8 : (dim <= 128 ? 16 : 32));   // key channels per thread: dim / 8 lanes, rounded up to a float4
  const size_t stage_floats = (size_t)kScanTok * kScanLanes * (dpt + 4) * (decay_mode >= 2 ? 3 : 2) + kScanTok * kScanCols + 2 * kScanTok;
  const size_t smem = 2 * stage_floats * sizeof(float);
  dim3 grid((vdim + kScanCols - 1) / kScanCols, H, portions);
  const int threads = kScanCols / 2 * kScanLanes;
  auto al16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec = dim % 4 == 0 && vdim % 4 == 0 && ldq % 4 == 0 && ldk % 4 == 0 && ldv % 4 == 0 && al16(q) && al16(k) && al16(v) &&
                   (decay_mode < 2 || (lda % 4 == 0 && al16(a)));
#define OMC_SCAN_LAUNCH(DPT, VEC)                                                                                        \
  do {                                                                                                                   \
    static bool attr_done[kMaxDevices] = {};                                                                             \
    if (!attr_done[cur_device()]) {                                                                                      \
      cudaFuncSetAttribute(linear_state_scan_kernel<DPT, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024); \
      attr_done[cur_device()] = true;                                                                                    \
    }                                                                                                                    \
    linear_state_scan_kernel<DPT, VEC><<<grid, threads, smem, st>>>(s);                                                  \
  } while (0)
#define OMC_SCAN_DPT(DPT)          \
  do {                             \
    if (vec) OMC_SCAN_LAUNCH(DPT, true); \
    else OMC_SCAN_LAUNCH(DPT, false);    \
  } while (0)
  if (dpt == 4) OMC_SCAN_DPT(4);
  else if (dpt == 8) OMC_SCAN_DPT(8);
  else if (dpt == 16) OMC_SCAN_DPT(16);
  else OMC_SCAN_DPT(32);
#undef OMC_SCAN_DPT
#undef OMC_SCAN_LAUNCH
  return check_launch("omc_linear_state_scan");
}

extern "C" int omc_gated_rms_rows(const float* x, long long ldx, int rows, int groups, int n, const void* w, int w_dt, float eps,
                                  const float* gate, long long ldg, int gate_act, void* y, int y_dt, long long ldy, void* stream) {
  if (x == nullptr || w == nullptr || y == nullptr || rows < 0 || groups <= 0 || n <= 0 || gate_act < 0 || gate_act > 2)
    return set_error(OMC_ERR_ARG, "omc_gated_rms_rows: bad argument");
  if (rows == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int gy = groups > 8 ? (groups + 7) / 8 : 1;
  OMC_DT_SWITCH(w_dt, TW, OMC_DT_SWITCH(y_dt, TY, {
    gated_rms_kernel<TW, TY><<<dim3(rows, gy > 65535 ? 65535 : gy), 256, 0, st>>>(x, ldx, groups, n, static_cast<const TW*>(w), eps,
                                                                                 gate, ldg, gate_act, static_cast<TY*>(y), ldy);
  }))
  return check_launch("omc_gated_rms_rows");
}

extern "C" int omc_map_rows(float* x, long long ldx, int rows, int cols, int op, const float* A_log, const float* bias, int group,
                            float p_exp, void* stream) {
  if (x == nullptr || rows < 0 || cols <= 0 || op < 1 || op > 3 || (op == 2 && (A_log == nullptr || bias == nullptr || group <= 0)))
    return set_error(OMC_ERR_ARG, "omc_map_rows: bad argument");
  if (rows == 0) return OMC_OK;
  const long long total = (long long)rows * cols;
  map_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, ldx, cols, total, op, A_log, bias, group, p_exp);
  return check_launch("omc_map_rows");
}

extern "C" int omc_dyt_conv(const float* x, long long ldx, const float* y1, long long ld1, float a1, const float* y2, long long ld2, float a2,
                            float* x_out, long long ldxo, const float* alpha, const void* nw, const void* nb, const void* cw, int w_dt,
                            int taps, const int32_t* pos, const int32_t* slot, float* state, void* u, int u_dt, long long ldu, int T, int C,
                            int single_rows, void* stream) {
  if (x == nullptr || alpha == nullptr || nw == nullptr || nb == nullptr || cw == nullptr || pos == nullptr || slot == nullptr || u == nullptr ||
      T < 0 || C <= 0 || taps < 1 || taps > kConvMaxTaps || (taps > 1 && state == nullptr) || ((y1 != nullptr || y2 != nullptr) && x_out == nullptr) ||
      (x_out == x && (y1 != nullptr || y2 != nullptr)))
    return set_error(OMC_ERR_ARG, "omc_dyt_conv: bad argument");
  if (T == 0) return OMC_OK;
  const int ch_block = C < 512 ? C : 512;
  const int blocks = (C + ch_block - 1) / ch_block;
  if (blocks > 65535) return set_error(OMC_ERR_SHAPE, "omc_dyt_conv: too many channel blocks");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rows_per_cta = T >= 256 ? kDytRows : 1;
  const size_t smem = (size_t)ch_block * (rows_per_cta + taps - 1) * sizeof(float);
  const float* xs = (y1 != nullptr || y2 != nullptr) ? x_out : x;   // where the save kernel finds the updated stream
  const long long ldxs = (y1 != nullptr || y2 != nullptr) ? ldxo : ldx;
  OMC_DT_SWITCH(w_dt, TW, OMC_DT_SWITCH(u_dt, TU, {
    if (smem > 48 * 1024) cudaFuncSetAttribute(dyt_conv_kernel<TW, TU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dyt_conv_kernel<TW, TU><<<dim3((T + rows_per_cta - 1) / rows_per_cta, blocks), 256, smem, st>>>(
        x, ldx, y1, ld1, a1, y2, ld2, a2, x_out, ldxo, alpha, static_cast<const TW*>(nw), static_cast<const TW*>(nb), static_cast<const TW*>(cw),
        taps, pos, slot, state, static_cast<TU*>(u), ldu, T, C, ch_block, rows_per_cta, single_rows ? 1 : 0);
    if (taps > 1 && !single_rows)
      dyt_state_save_kernel<is_bf16_t<TU>::value, TW><<<dim3(T, (C + 1023) / 1024), 256, 0, st>>>(xs, ldxs, alpha, static_cast<const TW*>(nw), static_cast<const TW*>(nb), C,
                                                                           taps - 1, T, pos, slot, state);
  }))
  return check_launch("omc_dyt_conv");
}

extern "C" int omc_selective_scan(const void* x, int x_dt, long long ldx, const float* dt, long long lddt, const float* dt_bias, const float* B,
                                  long long ldb, const float* Cm, long long ldc, const float* A_log, const float* D, const float* z, long long ldz,
                                  float* state, void* y, int y_dt, long long ldy, const int32_t* row_begin, int portions, const int32_t* pos,
                                  const int32_t* slot, int inner, int N, void* stream) {
  if (x == nullptr || dt == nullptr || dt_bias == nullptr || B == nullptr || Cm == nullptr || A_log == nullptr || D == nullptr || state == nullptr ||
      y == nullptr || row_begin == nullptr || pos == nullptr || slot == nullptr || portions < 0 || inner <= 0 || N <= 0)
    return set_error(OMC_ERR_ARG, "omc_selective_scan: bad argument");
  if (portions == 0) return OMC_OK;
  if (N > 256) return set_error(OMC_ERR_SHAPE, "omc_selective_scan: more than 256 states per channel");
  if (portions > 65535) return set_error(OMC_ERR_SHAPE, "omc_selective_scan: more than 65535 portions");
  if (x_dt != y_dt) return set_error(OMC_ERR_ARG, "omc_selective_scan: x and y must have the same dtype");
  SelArgs s{x, ldx, dt, lddt, dt_bias, B, ldb, Cm, ldc, A_log, D, z, ldz, state, y, ldy, row_begin, pos, slot, inner, N};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // two states per lane up to 64 states (many short dependency chains: the loop over tokens is sequential), eight above
  const int per = N <= 64 ? 2 : 8;
  int lanes = 1;
  while (lanes * per < N) lanes <<= 1;
  const int ch = kSelThreads / lanes;
  const size_t smem = sizeof(float) * ((size_t)3 * kSelTok * ch + 2 * (size_t)kSelTok * N);
  dim3 grid((inner + ch - 1) / ch, portions);
#define OMC_SEL_LAUNCH(L, P)                                                        \
  OMC_DT_SWITCH(x_dt, TD, {                                                         \
    selective_scan_kernel<L, P, TD><<<grid, kSelThreads, smem, st>>>(s);            \
  })
  if (per == 2) {
    if (lanes == 1) { OMC_SEL_LAUNCH(1, 2) }
    else if (lanes == 2) { OMC_SEL_LAUNCH(2, 2) }
    else if (lanes == 4) { OMC_SEL_LAUNCH(4, 2) }
    else if (lanes == 8) { OMC_SEL_LAUNCH(8, 2) }
    else if (lanes == 16) { OMC_SEL_LAUNCH(16, 2) }
    else { OMC_SEL_LAUNCH(32, 2) }
  } else {
    if (lanes == 16) { OMC_SEL_LAUNCH(16, 8) }
    else { OMC_SEL_LAUNCH(32, 8) }
  }
#undef OMC_SEL_LAUNCH
  return check_launch("omc_selective_scan");
}
