// Mixture-of-experts routing with a score correction and identity experts, the expert-sorted row layout, and the combine that is
// fused with the output-side norm and the residual add.
//
//   router:   s = softmax(z + bias) over ALL router outputs (experts, then identity experts); the choice is made on s + correction, the
//             mixing weights are the uncorrected s of the chosen outputs - as they are, or divided by their sum (`renorm`), which is
//             the softmax over the chosen logits alone. An identity expert returns its input,
//             has no weights and takes no rows in the sorted layout. The shared expert's gate logit rides as one more column of z.
//   plan:     one CTA: segment starts padded to whole row tiles, tile -> expert table, counters reset for the next call.
//   scatter:  one CTA per row: the row is copied to a place in the segment of each chosen expert (atomic cursor per expert; the
//             place a row gets does not affect its result).
//   combine:  y = sum_j w_j * (expert output | the row itself) + gate * shared output, then x <- x + y / rms(y) * (1 + g) and the
//             rounded copy for the next sublayer - one pass, the row lives in shared memory.
// No host synchronisation: the block can be captured in a CUDA graph.
#include "seq_common.cuh"

namespace omc {

constexpr int kRouteWarps = 4;

// One warp per row. Shared memory per warp: s[E_tot] (softmax scores) and ch[E_tot] (choice values, -inf once taken).
__global__ void __launch_bounds__(kRouteWarps * 32) router_topk_kernel(const float* __restrict__ z, long long ldz, int T, int E_tot,
                                                                       int experts, int top, const float* __restrict__ correction,
                                                                       const float* __restrict__ bias, int renorm, int score,
                                                                       int has_gate, int32_t* __restrict__ ids, float* __restrict__ w,
                                                                       float* __restrict__ gate, int32_t* __restrict__ counts) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + warp;
  if (t >= T) return;
  float* s = sm + (size_t)warp * 2 * E_tot;
  float* ch = s + E_tot;
  const float* zr = z + (long long)t * ldz;
  float mx = -INFINITY;
  for (int e = lane; e < E_tot; e += 32) {
    const float v = bias != nullptr ? zr[e] + bias[e] : zr[e];
    ch[e] = v;   // the logit with its bias; replaced by the choice value below
    mx = fmaxf(mx, v);
  }
  mx = seq_warp_max(mx);
  if (score == OMC_ROUTER_SIGMOID) {   // every output scored on its own; the sigmoid is monotonic, so the logits choose
    for (int e = lane; e < E_tot; e += 32) {
      const float p = 1.f / (1.f + expf(-ch[e]));
      s[e] = p;
      if (correction != nullptr) ch[e] = p + correction[e];
    }
  } else {
    float sum = 0.f;
    for (int e = lane; e < E_tot; e += 32) {
      const float p = expf(ch[e] - mx);
      s[e] = p;
      sum += p;
    }
    sum = seq_warp_sum(sum);
    const float inv = 1.f / sum;
    for (int e = lane; e < E_tot; e += 32) {
      const float p = s[e] * inv;
      s[e] = p;
      if (correction != nullptr) ch[e] = p + correction[e];   // without a correction the choice is made on the logits themselves
    }
  }
  __syncwarp();
  for (int k = 0; k < top; ++k) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
    for (int e = lane; e < E_tot; e += 32) {
      const float v = ch[e];
      if (v > bv) {  // ascending e per lane: the lowest index wins a tie
        bv = v;
        be = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) {
        bv = ov;
        be = oe;
      }
    }
    if (be >= E_tot) be = k % E_tot;  // only with NaN logits: stay inside the tables
    if (lane == 0) {
      ids[(long long)t * top + k] = be;
      w[(long long)t * top + k] = s[be];
      if (be < experts) atomicAdd(counts + be, 1);
      ch[be] = -INFINITY;
    }
    __syncwarp();
  }
  if (renorm && lane == 0) {   // softmax over the chosen alone: exp(z - max) / sum over the chosen, the common factor cancels
    float tot = 0.f;
    for (int k = 0; k < top; ++k) tot += w[(long long)t * top + k];
    const float r = 1.f / tot;
    for (int k = 0; k < top; ++k) w[(long long)t * top + k] *= r;
  }
  if (has_gate && lane == 0) gate[t] = 1.f / (1.f + expf(-zr[E_tot]));
}

__global__ void __launch_bounds__(256) moe_plan_tiles_kernel(int32_t* __restrict__ counts, int experts, int tile, int max_tiles,
                                                             int32_t* __restrict__ seg_start, int32_t* __restrict__ cursor,
                                                             int32_t* __restrict__ tile_group) {
  for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) tile_group[i] = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    int tiles = 0;
    for (int e = 0; e < experts; ++e) {
      const int n = (counts[e] + tile - 1) / tile;
      seg_start[e] = tiles * tile;
      for (int i = 0; i < n && tiles + i < max_tiles; ++i) tile_group[tiles + i] = e;
      tiles += n;
    }
    seg_start[experts] = tiles * tile;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    counts[e] = 0;
    cursor[e] = 0;
  }
}

template <typename TT>
__global__ void __launch_bounds__(128) moe_scatter_rows_kernel(const TT* __restrict__ x, long long ldx, int C,
                                                               const int32_t* __restrict__ ids, int top, int experts,
                                                               const int32_t* __restrict__ seg_start, int32_t* __restrict__ cursor,
                                                               int32_t* __restrict__ slot_of, TT* __restrict__ xs, long long ldxs,
                                                               const float* __restrict__ row_w) {
  __shared__ int s_slot[32];
  const int t = blockIdx.x;
  if (threadIdx.x < top) {
    const int e = ids[(long long)t * top + threadIdx.x];
    int sl = -1;
    if (e < experts) sl = seg_start[e] + atomicAdd(cursor + e, 1);
    s_slot[threadIdx.x] = sl;
    slot_of[(long long)t * top + threadIdx.x] = sl;
  }
  __syncthreads();
  for (int k = 0; k < top; ++k) {
    const int sl = s_slot[k];
    if (sl < 0) continue;
    if (row_w != nullptr) {   // the mixing weight multiplies the expert's INPUT
      const float wk = row_w[(long long)t * top + k];
      for (int c = threadIdx.x; c < C; c += blockDim.x) stf(xs + (long long)sl * ldxs + c, wk * ldf(x + (long long)t * ldx + c));
    } else {
      for (int c = threadIdx.x; c < C; c += blockDim.x) xs[(long long)sl * ldxs + c] = x[(long long)t * ldx + c];
    }
  }
}

// plan + scatter of a small step (decode rows) in ONE single-CTA launch: segment starts and the tile table as in the plan kernel,
// then row after row is copied to its places (the cursors live in shared memory).
template <typename TT>
__global__ void __launch_bounds__(256) moe_plan_scatter_small_kernel(int32_t* __restrict__ counts, int experts, int tile, int max_tiles,
                                                                     int32_t* __restrict__ seg_start, int32_t* __restrict__ tile_group,
                                                                     const TT* __restrict__ x, long long ldx, int T, int C,
                                                                     const int32_t* __restrict__ ids, int top,
                                                                     int32_t* __restrict__ slot_of, TT* __restrict__ xs, long long ldxs,
                                                                     const float* __restrict__ row_w) {
  extern __shared__ int32_t s_seg[];  // [experts]: next free row of every expert's segment
  __shared__ int s_slot[32];
  for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) tile_group[i] = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    int tiles = 0;
    for (int e = 0; e < experts; ++e) {
      const int n = (counts[e] + tile - 1) / tile;
      seg_start[e] = tiles * tile;
      s_seg[e] = tiles * tile;
      for (int i = 0; i < n && tiles + i < max_tiles; ++i) tile_group[tiles + i] = e;
      tiles += n;
      counts[e] = 0;
    }
    seg_start[experts] = tiles * tile;
  }
  __syncthreads();
  for (int t = 0; t < T; ++t) {
    if (threadIdx.x == 0) {
      for (int k = 0; k < top; ++k) {
        const int e = ids[(long long)t * top + k];
        const int sl = e < experts ? s_seg[e]++ : -1;
        s_slot[k] = sl;
        slot_of[(long long)t * top + k] = sl;
      }
    }
    __syncthreads();
    for (int k = 0; k < top; ++k) {
      const int sl = s_slot[k];
      if (sl < 0) continue;
      const float wk = row_w != nullptr ? row_w[(long long)t * top + k] : 1.f;
      if (row_w != nullptr) {
        for (int c = threadIdx.x; c < C; c += blockDim.x) stf(xs + (long long)sl * ldxs + c, wk * ldf(x + (long long)t * ldx + c));
      } else {
        for (int c = threadIdx.x; c < C; c += blockDim.x) xs[(long long)sl * ldxs + c] = x[(long long)t * ldx + c];
      }
    }
    __syncthreads();
  }
}

template <typename TW, typename TB>
__global__ void __launch_bounds__(256) moe_combine_norm_kernel(const float* __restrict__ ys, long long ldys,
                                                               const int32_t* __restrict__ slot_of, const float* __restrict__ w, int top,
                                                               const float* __restrict__ gate, const float* __restrict__ ysh,
                                                               long long ldysh, const TW* __restrict__ nw, float eps,
                                                               float* __restrict__ h32, long long ldh, const TW* __restrict__ w_next,
                                                               TB* __restrict__ xb, long long ldxb, int C) {
  extern __shared__ float srow[];  // y [C]
  __shared__ float red[33];
  __shared__ int s_slot[32];
  __shared__ float s_w[32];
  const int t = blockIdx.x;
  if (threadIdx.x < top) {
    s_slot[threadIdx.x] = slot_of[(long long)t * top + threadIdx.x];
    s_w[threadIdx.x] = w[(long long)t * top + threadIdx.x];
  }
  __syncthreads();
  const float g = (gate != nullptr && ysh != nullptr) ? gate[t] : 0.f;
  float* hr = h32 + (long long)t * ldh;
  float ss = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float y = 0.f;
    for (int k = 0; k < top; ++k) {
      const int sl = s_slot[k];
      y = fmaf(s_w[k], sl >= 0 ? ys[(long long)sl * ldys + c] : hr[c], y);
    }
    if (ysh != nullptr) y = fmaf(g, ysh[(long long)t * ldysh + c], y);
    srow[c] = y;
    ss = fmaf(y, y, ss);
  }
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)C + eps);
  float sh = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = hr[c] + srow[c] * rstd * (1.f + ldf(nw + c));
    hr[c] = v;
    srow[c] = v;
    sh = fmaf(v, v, sh);
    if (xb != nullptr && w_next == nullptr) stf(xb + (long long)t * ldxb + c, v);
  }
  if (xb == nullptr || w_next == nullptr) return;
  sh = block_sum(sh, red);   // the next sublayer reads the row normed: x / rms(x) * (1 + w_next)
  const float rn = 1.f / sqrtf(sh / (float)C + eps);
  for (int c = threadIdx.x; c < C; c += blockDim.x) stf(xb + (long long)t * ldxb + c, srow[c] * rn * (1.f + ldf(w_next + c)));
}


// Combine + residual + depth-weighted average of the layer outputs, one pass over the row:
//   y = sum_j (w[t, j] or 1) * ys[slot_of[t, j]]            (ys NULL: no feed-forward, y = 0)
//   xn = x[t] + a1 * y1[t] + a2 * y2[t] + mult * y           -> streams[n_streams - 1][t]   (this layer's result; y1 / y2: sublayer
//                                                               outputs that have not entered the stream yet, NULL: none)
//   out[t] = sum_{j < n_streams} coef[j] * streams[j][t]     (coef NULL: out = xn)
// streams[j] = streams + j * stream_stride: the embedding output and every earlier layer's result.
template <typename TW>
__global__ void __launch_bounds__(256) moe_combine_depth_kernel(const float* __restrict__ ys, long long ldys, const int32_t* __restrict__ slot_of,
                                                                const float* __restrict__ w, int top, const float* __restrict__ x,
                                                                long long ldx, const float* __restrict__ y1, long long ld1, float a1,
                                                                const float* __restrict__ y2, long long ld2, float a2, float mult,
                                                                float* __restrict__ streams,
                                                                long long stream_stride, long long lds, int n_streams,
                                                                const TW* __restrict__ coef, float* __restrict__ out, long long ldo, int C) {
  __shared__ int s_slot[32];
  __shared__ float s_w[32];
  const long long t = blockIdx.x;
  if (ys != nullptr && threadIdx.x < top) {
    s_slot[threadIdx.x] = slot_of[t * top + threadIdx.x];
    s_w[threadIdx.x] = w != nullptr ? w[t * top + threadIdx.x] : 1.f;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float xn = x[t * ldx + c];
    if (y1 != nullptr) xn = fmaf(a1, y1[t * ld1 + c], xn);
    if (y2 != nullptr) xn = fmaf(a2, y2[t * ld2 + c], xn);
    if (ys != nullptr) {
      float y = 0.f;
      for (int k = 0; k < top; ++k) {
        const int sl = s_slot[k];
        if (sl >= 0) y = fmaf(s_w[k], ys[(long long)sl * ldys + c], y);
      }
      xn = fmaf(mult, y, xn);
    }
    if (streams != nullptr) streams[(long long)(n_streams - 1) * stream_stride + t * lds + c] = xn;
    float o = xn;
    if (coef != nullptr) {
      o = 0.f;
      for (int j = 0; j + 1 < n_streams; ++j) o = fmaf(ldf(coef + j), streams[(long long)j * stream_stride + t * lds + c], o);
      o = fmaf(ldf(coef + n_streams - 1), xn, o);
    }
    out[t * ldo + c] = o;
  }
}

}  // namespace omc

using namespace omc;

extern "C" int omc_router_topk(const float* z, long long ldz, int T, int E_tot, int experts, int top, const float* correction,
                               const float* bias, int renorm, int score, int has_gate, int32_t* ids, float* w, float* gate, int32_t* counts,
                               void* stream) {
  if (score != OMC_ROUTER_SOFTMAX && score != OMC_ROUTER_SIGMOID) return set_error(OMC_ERR_ARG, "omc_router_topk: unknown score function");
  if (z == nullptr || ids == nullptr || w == nullptr || counts == nullptr || T < 0 || E_tot <= 0 || experts < 0 || experts > E_tot ||
      top <= 0 || top > E_tot || (has_gate && gate == nullptr))
    return set_error(OMC_ERR_ARG, "omc_router_topk: bad argument");
  if (E_tot > 4096 || top > 32) return set_error(OMC_ERR_SHAPE, "omc_router_topk: more than 4096 router outputs or top above 32");
  if (T == 0) return OMC_OK;
  const size_t smem = sizeof(float) * 2 * (size_t)E_tot * kRouteWarps;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(router_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error(OMC_ERR_CUDA, cudaGetErrorString(e));
  }
  router_topk_kernel<<<(T + kRouteWarps - 1) / kRouteWarps, kRouteWarps * 32, smem, static_cast<cudaStream_t>(stream)>>>(
      z, ldz, T, E_tot, experts, top, correction, bias, renorm, score, has_gate, ids, w, gate, counts);
  return check_launch("omc_router_topk");
}

extern "C" int omc_moe_plan_tiles(int32_t* counts, int experts, int tile, int max_tiles, int32_t* seg_start, int32_t* cursor,
                                  int32_t* tile_group, void* stream) {
  if (counts == nullptr || seg_start == nullptr || cursor == nullptr || tile_group == nullptr || experts <= 0 || tile <= 0 || max_tiles <= 0)
    return set_error(OMC_ERR_ARG, "omc_moe_plan_tiles: bad argument");
  moe_plan_tiles_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(counts, experts, tile, max_tiles, seg_start, cursor, tile_group);
  return check_launch("omc_moe_plan_tiles");
}

extern "C" int omc_moe_scatter_rows(const void* x, int dt, long long ldx, int T, int C, const int32_t* ids, int top, int experts,
                                    const int32_t* seg_start, int32_t* cursor, int32_t* slot_of, void* xs, long long ldxs, const float* row_w,
                                    void* stream) {
  if (x == nullptr || ids == nullptr || seg_start == nullptr || cursor == nullptr || slot_of == nullptr || xs == nullptr || T < 0 ||
      C <= 0 || top <= 0 || top > 32)
    return set_error(OMC_ERR_ARG, "omc_moe_scatter_rows: bad argument");
  if (T == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(dt, TT, {
    moe_scatter_rows_kernel<TT><<<T, 128, 0, st>>>(static_cast<const TT*>(x), ldx, C, ids, top, experts, seg_start, cursor, slot_of,
                                                   static_cast<TT*>(xs), ldxs, row_w);
  })
  return check_launch("omc_moe_scatter_rows");
}

extern "C" int omc_moe_plan_scatter_small(int32_t* counts, int experts, int tile, int max_tiles, int32_t* seg_start, int32_t* tile_group,
                                          const void* x, int dt, long long ldx, int T, int C, const int32_t* ids, int top, int32_t* slot_of,
                                          void* xs, long long ldxs, const float* row_w, void* stream) {
  if (counts == nullptr || seg_start == nullptr || tile_group == nullptr || x == nullptr || ids == nullptr || slot_of == nullptr ||
      xs == nullptr || experts <= 0 || experts > 8192 || tile <= 0 || max_tiles <= 0 || T < 0 || C <= 0 || top <= 0 || top > 32)
    return set_error(OMC_ERR_ARG, "omc_moe_plan_scatter_small: bad argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(dt, TT, {
    moe_plan_scatter_small_kernel<TT><<<1, 256, experts * sizeof(int32_t), st>>>(counts, experts, tile, max_tiles, seg_start, tile_group,
                                                                                static_cast<const TT*>(x), ldx, T, C, ids, top, slot_of,
                                                                                static_cast<TT*>(xs), ldxs, row_w);
  })
  return check_launch("omc_moe_plan_scatter_small");
}

extern "C" int omc_moe_combine_norm(const float* ys, long long ldys, const int32_t* slot_of, const float* w, int top, const float* gate,
                                    const float* ysh, long long ldysh, const void* nw, int nw_dt, float eps, float* h32, long long ldh,
                                    const void* w_next, void* xb, int xb_dt, long long ldxb, int T, int C, void* stream) {
  if (slot_of == nullptr || w == nullptr || nw == nullptr || h32 == nullptr || T < 0 || C <= 0 || top <= 0 || top > 32)
    return set_error(OMC_ERR_ARG, "omc_moe_combine_norm: bad argument");
  if (T == 0) return OMC_OK;
  if ((size_t)C * sizeof(float) > 200 * 1024) return set_error(OMC_ERR_SHAPE, "omc_moe_combine_norm: row wider than 51200");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)C * sizeof(float);
  OMC_DT_SWITCH(nw_dt, TW, OMC_DT_SWITCH(xb_dt, TB, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(moe_combine_norm_kernel<TW, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return set_error(OMC_ERR_CUDA, cudaGetErrorString(e));
    }
    moe_combine_norm_kernel<TW, TB><<<T, 256, smem, st>>>(ys, ldys, slot_of, w, top, gate, ysh, ldysh, static_cast<const TW*>(nw), eps,
                                                          h32, ldh, static_cast<const TW*>(w_next), static_cast<TB*>(xb), ldxb, C);
  }))
  return check_launch("omc_moe_combine_norm");
}

extern "C" int omc_moe_combine_depth(const float* ys, long long ldys, const int32_t* slot_of, const float* w, int top, const float* x,
                                     long long ldx, const float* y1, long long ld1, float a1, const float* y2, long long ld2, float a2,
                                     float mult, float* streams, long long stream_stride, long long lds, int n_streams,
                                     const void* coef, int coef_dt, float* out, long long ldo, int T, int C, void* stream) {
  if (x == nullptr || out == nullptr || T < 0 || C <= 0 || (ys != nullptr && (slot_of == nullptr || top <= 0 || top > 32)) ||
      (coef != nullptr && (streams == nullptr || n_streams < 1)) || (streams != nullptr && n_streams < 1))
    return set_error(OMC_ERR_ARG, "omc_moe_combine_depth: bad argument");
  if (T == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(coef_dt, TW, {
    moe_combine_depth_kernel<TW><<<T, 256, 0, st>>>(ys, ldys, slot_of, w, top, x, ldx, y1, ld1, a1, y2, ld2, a2, mult, streams, stream_stride, lds, n_streams,
                                                    static_cast<const TW*>(coef), out, ldo, C);
  })
  return check_launch("omc_moe_combine_depth");
}
