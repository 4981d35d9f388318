// Mixture of clipped-GLU experts: fp32 softmax router with top-k choice, and the expert products for a handful of
// tokens (decode, short portions) as matrix-vector kernels that read the expert index from device memory — no host
// round trip, so the step can be captured into a CUDA graph.  Prompt-sized batches sort their rows by expert and use
// the gather / scatter kernels at the end of this file around library GEMMs.
#include "lm_common.cuh"

#include <type_traits>

using namespace lm;

namespace {

constexpr int kWarps = 8;

// one warp: scores = softmax over z[0..E) (shared memory, destroyed), then the `top` largest as they are (ties: lowest index)
__device__ __forceinline__ void softmax_topk(float* z, int E, int top, int lane, int32_t* idx_out, float* weight_out) {
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float den = 0.f;
  for (int e = lane; e < E; e += 32) den += expf(z[e] - mx);
  den = warp_sum(den);
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = E;
    for (int e = lane; e < E; e += 32)
      if (z[e] > best) best = z[e], at = e;          // ascending e: the lowest index wins inside a lane
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, at, o);
      if (ov > best || (ov == best && oi < at)) best = ov, at = oi;
    }
    if (lane == 0) {
      idx_out[k] = at;
      weight_out[k] = expf(best - mx) / den;
    }
    __syncwarp();
    if (lane == 0 && at < E) z[at] = -INFINITY;
    __syncwarp();
  }
}

// one CTA per token: E dot products (a warp each, round robin), then warp 0 does softmax + top-k.  A step of few tokens
// has few CTAs: each then runs 32 warps, so that one token's router matrix is read by more loads in flight.
template <typename T>
__global__ void __launch_bounds__(1024) router_topk_kernel(const T* __restrict__ h, const T* __restrict__ wr, int64_t W, int E, int top,
                                   int32_t* __restrict__ idx, float* __restrict__ weight) {
  extern __shared__ float sm[];
  float* xs = sm;          // [W]
  float* z = sm + W;       // [E]
  const int64_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  stage_f32(h + t * W, xs, W);
  __syncthreads();
  const bool vec = rows_vectorizable<T>(wr, W);
  const int nw = (int)(blockDim.x >> 5);
  bool done = false;
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    if (vec) {   // a warp's experts two at a time
      for (int e = warp; e < E; e += 2 * nw) {
        const int e2 = e + nw < E ? e + nw : e;
        const T* const rows[2] = {wr + (int64_t)e * W, wr + (int64_t)e2 * W};
        const float* const xr[2] = {xs, xs};
        float v[2];
        warp_dot_rows<2, 4>(rows, xr, e + nw < E ? 2 : 1, W, lane, v);
        if (lane == 0) {
          z[e] = v[0];
          if (e + nw < E) z[e2] = v[1];
        }
      }
      done = true;
    }
  }
  if (!done) {
    for (int e = warp; e < E; e += nw) {
      const float v = warp_dot(wr + (int64_t)e * W, xs, W, lane, vec);
      if (lane == 0) z[e] = v;
    }
  }
  __syncthreads();
  if (warp != 0) return;
  softmax_topk(z, E, top, lane, idx + t * top, weight + t * top);
}

// one warp per token over logits a GEMM has made (prompt portions: the router matrix is read once, not once per token)
__global__ void router_topk_logits_kernel(const float* __restrict__ logits, int64_t n, int E, int top,
                                          int32_t* __restrict__ idx, float* __restrict__ weight) {
  extern __shared__ float sm[];   // [kWarps][E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * kWarps + warp;
  if (t >= n) return;
  float* z = sm + (size_t)warp * E;
  for (int e = lane; e < E; e += 32) z[e] = logits[t * E + e];
  __syncwarp();
  softmax_topk(z, E, top, lane, idx + t * top, weight + t * top);
}

// Sigmoid router with a selection correction and group-limited choice, one warp per token over fp32 logits:
//   s_e = sigmoid(z_e); the choice is made on c_e = s_e + correction_e.  The experts form n_groups equal groups of
//   neighbours; a group's score is the sum of its two largest c (of its only one, for groups of one); only experts of
//   the `keep` best groups can be chosen (the others count as -inf); the `top` largest c win (ties: lowest index);
//   weight = s_e / (sum of the chosen s + 1e-20) * scale.
// Shared memory per warp: s [E], c [E], group scores [n_groups].
__global__ void router_group_topk_kernel(const float* __restrict__ logits, int64_t n, int E, int top,
                                         const float* __restrict__ correction, int n_groups, int keep, float scale,
                                         int32_t* __restrict__ idx, float* __restrict__ weight) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * kWarps + warp;
  if (t >= n) return;
  float* s = sm + (size_t)warp * (2 * E + n_groups);
  float* c = s + E;
  float* gs = c + E;
  for (int e = lane; e < E; e += 32) {
    const float v = 1.f / (1.f + expf(-logits[t * E + e]));
    s[e] = v;
    c[e] = v + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  const int per = E / n_groups;
  if (keep < n_groups) {
    for (int g = lane; g < n_groups; g += 32) {
      float b0 = -INFINITY, b1 = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float v = c[e];
        if (v > b0) b1 = b0, b0 = v;
        else if (v > b1) b1 = v;
      }
      gs[g] = per > 1 ? b0 + b1 : b0;
    }
    __syncwarp();
    // every group but the `keep` best loses its experts: take the worst n_groups - keep out one by one (ties: the
    // higher index goes first, so the lower index stays)
    for (int r = 0; r < n_groups - keep; ++r) {
      float worst = INFINITY;
      int at = -1;
      for (int g = lane; g < n_groups; g += 32) {
        const float v = gs[g];
        if (v <= worst && v != INFINITY) worst = v, at = g;      // ascending g: the highest index wins inside a lane
      }
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, worst, o);
        const int oi = __shfl_xor_sync(0xffffffffu, at, o);
        if (oi >= 0 && (at < 0 || ov < worst || (ov == worst && oi > at))) worst = ov, at = oi;
      }
      if (at >= 0) {
        for (int e = at * per + lane; e < (at + 1) * per; e += 32) c[e] = -INFINITY;
        if (lane == 0) gs[at] = INFINITY;   // out of the running
      }
      __syncwarp();
    }
  }
  float sum = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = E;
    for (int e = lane; e < E; e += 32)
      if (c[e] > best) best = c[e], at = e;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, at, o);
      if (ov > best || (ov == best && oi < at)) best = ov, at = oi;
    }
    if (at >= E) at = 0;   // fewer candidates than `top`: cannot happen for top <= keep * per
    const float sv = s[at];
    sum += sv;
    if (lane == 0) {
      idx[t * top + k] = at;
      weight[t * top + k] = sv;
    }
    __syncwarp();
    if (lane == 0) c[at] = -INFINITY;
    __syncwarp();
  }
  const float k = scale / (sum + 1e-20f);
  __syncwarp();
  for (int j = lane; j < top; j += 32) weight[t * top + j] *= k;
}

// grid (ceil(ff / 8), pairs): a warp computes one row of both projections of its pair's expert
template <typename T>
__global__ void expert_gate_up_kernel(const T* __restrict__ h, const T* __restrict__ wg, const T* __restrict__ wu,
                                      const int32_t* __restrict__ idx, int top, int64_t W, int64_t ff,
                                      int64_t expert_stride, float limit, float alpha, float shift, T* __restrict__ y) {
  extern __shared__ float xs[];   // [W]
  const int64_t p = blockIdx.y, t = p / top;
  const int64_t e = idx ? idx[p] : 0;
  stage_f32(h + t * W, xs, W);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t f = (int64_t)blockIdx.x * kWarps + warp;
  if (f >= ff) return;
  const bool vec = rows_vectorizable<T>(wg, W) && rows_vectorizable<T>(wu, W);
  float a, b;
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    if (vec) {   // both rows together, four vectors each in flight
      const T* const rows[2] = {wg + e * expert_stride + f * W, wu + e * expert_stride + f * W};
      const float* const xr[2] = {xs, xs};
      float ab[2];
      warp_dot_rows<2, 4>(rows, xr, 2, W, lane, ab);
      a = ab[0], b = ab[1];
    } else {
      a = warp_dot(wg + e * expert_stride + f * W, xs, W, lane, false);
      b = warp_dot(wu + e * expert_stride + f * W, xs, W, lane, false);
    }
  } else {
    a = warp_dot(wg + e * expert_stride + f * W, xs, W, lane, vec);
    b = warp_dot(wu + e * expert_stride + f * W, xs, W, lane, vec);
  }
  if (lane == 0) {
    // the projections' outputs are activations of the storage type: round them as a GEMM would
    T ra, rb;
    stf(&ra, a);
    stf(&rb, b);
    const float g = fminf(ldf(&ra), limit);
    const float u = fminf(fmaxf(ldf(&rb), -limit), limit);
    stf(y + p * ff + f, g / (1.f + expf(-alpha * g)) * (u + shift));
  }
}

// grid (ceil(W / 8), n): a warp computes one output coordinate of its token over the token's `top` experts
template <typename T>
__global__ void expert_down_kernel(const T* __restrict__ y, const T* __restrict__ wd, const int32_t* __restrict__ idx,
                                   const float* __restrict__ weight, int top, int64_t W, int64_t ff, int accumulate,
                                   float* __restrict__ out) {
  extern __shared__ float ys[];   // [top][ff]
  const int64_t t = blockIdx.y;
  stage_f32(y + t * top * ff, ys, (int64_t)top * ff);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * kWarps + warp;
  if (w >= W) return;
  const bool vec = rows_vectorizable<T>(wd, ff);
  float acc = 0.f;
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    if (vec) {   // the rows of up to four of the token's experts together, two vectors each in flight
      for (int k0 = 0; k0 < top; k0 += 4) {
        const int kn = min(4, top - k0);
        const T* rows[4];
        const float* yr[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k = k0 + (j < kn ? j : 0);
          const int64_t e = idx ? idx[t * top + k] : 0;
          rows[j] = wd + (e * W + w) * ff;
          yr[j] = ys + (int64_t)k * ff;
        }
        const T* const rc[4] = {rows[0], rows[1], rows[2], rows[3]};
        const float* const yc[4] = {yr[0], yr[1], yr[2], yr[3]};
        float d[4];
        warp_dot_rows<4, 2>(rc, yc, kn, ff, lane, d);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (j < kn) {
            T rd;
            stf(&rd, d[j]);       // an expert's output is an activation of the storage type
            acc = fmaf(weight ? weight[t * top + k0 + j] : 1.f, ldf(&rd), acc);
          }
        }
      }
      if (lane == 0) out[t * W + w] = (accumulate ? out[t * W + w] : 0.f) + acc;
      return;
    }
  }
  for (int k = 0; k < top; ++k) {
    const int64_t e = idx ? idx[t * top + k] : 0;
    const float d = warp_dot(wd + (e * W + w) * ff, ys + (int64_t)k * ff, ff, lane, vec);
    T rd;
    stf(&rd, d);                  // an expert's output is an activation of the storage type
    acc = fmaf(weight ? weight[t * top + k] : 1.f, ldf(&rd), acc);
  }
  if (lane == 0) out[t * W + w] = (accumulate ? out[t * W + w] : 0.f) + acc;
}

// Top-k on the raw logits, weights = softmax over the chosen logits only.  One warp per token over fp32 logits[n][ld] that
// a GEMM has made; bias (fp32 [E]; null: none) is added first.  Column `extra` of the same row (>= 0) is a gate logit that
// rode along in the GEMM: extra_out[t] = sigmoid(logits[t][extra]).
__global__ void router_topk_renorm_kernel(const float* __restrict__ logits, int64_t ld, const float* __restrict__ bias, int64_t n,
                                          int E, int top, int extra, int32_t* __restrict__ idx, float* __restrict__ weight,
                                          float* __restrict__ extra_out) {
  extern __shared__ float sm[];   // [kWarps][E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * kWarps + warp;
  if (t >= n) return;
  float* z = sm + (size_t)warp * E;
  for (int e = lane; e < E; e += 32) z[e] = logits[t * ld + e] + (bias ? bias[e] : 0.f);
  if (extra >= 0 && lane == 0) extra_out[t] = 1.f / (1.f + expf(-logits[t * ld + extra]));
  __syncwarp();
  float first = 0.f, den = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = E;
    for (int e = lane; e < E; e += 32)
      if (z[e] > best) best = z[e], at = e;          // ascending e: the lowest index wins inside a lane
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, at, o);
      if (ov > best || (ov == best && oi < at)) best = ov, at = oi;
    }
    if (k == 0) first = best;                        // the largest logit: the softmax's reference point
    const float p = expf(best - first);
    den += p;
    if (lane == 0) {
      idx[t * top + k] = at;
      weight[t * top + k] = p;                       // divided by the sum below
      if (at < E) z[at] = -INFINITY;
    }
    __syncwarp();
  }
  for (int j = lane; j < top; j += 32) weight[t * top + j] /= den;
}

// grid (ceil(ff / 8), pairs): a warp computes one row of the up projection of its pair's expert; the unit has no gate:
// y = act(w_up[e] h), act 0: the square of relu.
template <typename T>
__global__ void expert_up_act_kernel(const T* __restrict__ h, const T* __restrict__ wu, const int32_t* __restrict__ idx, int top,
                                     int64_t W, int64_t ff, int64_t expert_stride, int act, T* __restrict__ y) {
  extern __shared__ float xs[];   // [W]
  const int64_t p = blockIdx.y, t = p / top;
  const int64_t e = idx ? idx[p] : 0;
  stage_f32(h + t * W, xs, W);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t f = (int64_t)blockIdx.x * kWarps + warp;
  if (f >= ff) return;
  const bool vec = rows_vectorizable<T>(wu, W) && (expert_stride % (16 / (int)sizeof(T)) == 0);
  const float a = warp_dot(wu + e * expert_stride + f * W, xs, W, lane, vec);
  if (lane == 0) {
    T ra;
    stf(&ra, a);                  // the projection's output is an activation of the storage type: round it as a GEMM would
    const float r = fmaxf(ldf(&ra), 0.f);
    (void)act;
    stf(y + p * ff + f, r * r);
  }
}

template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ h, const int64_t* __restrict__ src, int top, int64_t W, T* __restrict__ xs) {
  const int64_t i = blockIdx.x, t = src[i] / top;
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) xs[i * W + w] = h[t * W + w];
}

template <typename T>
__global__ void scatter_add_rows_kernel(const T* __restrict__ y, const int64_t* __restrict__ src, const float* __restrict__ weight,
                                        int top, int64_t W, float* __restrict__ out) {
  const int64_t i = blockIdx.x, p = src[i], t = p / top;
  const float k = weight[p];
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) atomicAdd(out + t * W + w, k * ldf(y + i * W + w));
}

}  // namespace

extern "C" int ao_lm_router_topk(const void* h, const void* w_router, int dt, int64_t n, int64_t width, int E, int top,
                                 int32_t* idx, float* weight, void* stream) {
  LM_CHECK_ARG(h && w_router && idx && weight && n > 0 && width > 0 && E > 0 && top > 0 && top <= E);
  const size_t smem = (size_t)(width + E) * sizeof(float);
  if (smem > 200 * 1024) return AO_B200_ERR_UNSUPPORTED;
  LM_DISPATCH(dt, {
    auto kern = router_topk_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    kern<<<(unsigned)n, (n <= 64 ? 32 : kWarps) * 32, smem, lm_stream(stream)>>>(static_cast<const T*>(h), static_cast<const T*>(w_router), width,
                                                               E, top, idx, weight);
  });
  return lm_launch_status();
}

extern "C" int ao_lm_router_topk_logits(const float* logits, int64_t n, int E, int top, int32_t* idx, float* weight, void* stream) {
  LM_CHECK_ARG(logits && idx && weight && n > 0 && E > 0 && top > 0 && top <= E);
  const size_t smem = (size_t)kWarps * E * sizeof(float);
  if (smem > 48 * 1024) return AO_B200_ERR_UNSUPPORTED;
  router_topk_logits_kernel<<<(unsigned)((n + kWarps - 1) / kWarps), kWarps * 32, smem, lm_stream(stream)>>>(logits, n, E, top, idx,
                                                                                                           weight);
  return lm_launch_status();
}

extern "C" int ao_lm_router_group_topk_logits(const float* logits, int64_t n, int E, int top, const float* correction,
                                              int n_groups, int keep, float scale, int32_t* idx, float* weight, void* stream) {
  LM_CHECK_ARG(logits && idx && weight && n > 0 && E > 0 && top > 0 && n_groups > 0 && E % n_groups == 0);
  LM_CHECK_ARG(keep > 0 && keep <= n_groups && top <= keep * (E / n_groups));
  const size_t smem = (size_t)kWarps * (2 * E + n_groups) * sizeof(float);
  if (smem > 48 * 1024) return AO_B200_ERR_UNSUPPORTED;
  router_group_topk_kernel<<<(unsigned)((n + kWarps - 1) / kWarps), kWarps * 32, smem, lm_stream(stream)>>>(
      logits, n, E, top, correction, n_groups, keep, scale, idx, weight);
  return lm_launch_status();
}

extern "C" int ao_lm_expert_gate_up_shift(const void* h, const void* w_gate, const void* w_up, int dt, const int32_t* idx,
                                          int64_t n, int top, int64_t width, int64_t ff, int64_t expert_stride, float limit,
                                          float alpha, float shift, void* y, void* stream) {
  LM_CHECK_ARG(h && w_gate && w_up && y && n > 0 && top > 0 && width > 0 && ff > 0 && n * top <= 65535);
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return AO_B200_ERR_UNSUPPORTED;
  dim3 grid((unsigned)((ff + kWarps - 1) / kWarps), (unsigned)(n * top));
  LM_DISPATCH(dt, {
    auto kern = expert_gate_up_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    kern<<<grid, kWarps * 32, smem, lm_stream(stream)>>>(static_cast<const T*>(h), static_cast<const T*>(w_gate),
                                                        static_cast<const T*>(w_up), idx, top, width, ff, expert_stride, limit, alpha,
                                                        shift, static_cast<T*>(y));
  });
  return lm_launch_status();
}

extern "C" int ao_lm_expert_gate_up(const void* h, const void* w_gate, const void* w_up, int dt, const int32_t* idx, int64_t n,
                                    int top, int64_t width, int64_t ff, int64_t expert_stride, float limit, float alpha, void* y,
                                    void* stream) {
  return ao_lm_expert_gate_up_shift(h, w_gate, w_up, dt, idx, n, top, width, ff, expert_stride, limit, alpha, 1.f, y, stream);
}

extern "C" int ao_lm_expert_down(const void* y, const void* w_down, int dt, const int32_t* idx, const float* weight, int64_t n,
                                 int top, int64_t width, int64_t ff, int accumulate, float* out, void* stream) {
  LM_CHECK_ARG(y && w_down && out && n > 0 && top > 0 && width > 0 && ff > 0 && n <= 65535);
  const size_t smem = (size_t)top * ff * sizeof(float);
  if (smem > 200 * 1024) return AO_B200_ERR_UNSUPPORTED;
  dim3 grid((unsigned)((width + kWarps - 1) / kWarps), (unsigned)n);
  LM_DISPATCH(dt, {
    auto kern = expert_down_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    kern<<<grid, kWarps * 32, smem, lm_stream(stream)>>>(static_cast<const T*>(y), static_cast<const T*>(w_down), idx, weight, top,
                                                        width, ff, accumulate, out);
  });
  return lm_launch_status();
}

extern "C" int ao_lm_router_topk_renorm_logits(const float* logits, int64_t ld, const float* bias, int64_t n, int E, int top,
                                               int extra, int32_t* idx, float* weight, float* extra_out, void* stream) {
  LM_CHECK_ARG(logits && idx && weight && n > 0 && E > 0 && top > 0 && top <= E && ld >= E && (extra < 0 || (extra < ld && extra_out)));
  const size_t smem = (size_t)kWarps * E * sizeof(float);
  if (smem > 48 * 1024) return AO_B200_ERR_UNSUPPORTED;
  router_topk_renorm_kernel<<<(unsigned)((n + kWarps - 1) / kWarps), kWarps * 32, smem, lm_stream(stream)>>>(
      logits, ld, bias, n, E, top, extra, idx, weight, extra_out);
  return lm_launch_status();
}

extern "C" int ao_lm_expert_up_act(const void* h, const void* w_up, int dt, const int32_t* idx, int64_t n, int top, int64_t width,
                                   int64_t ff, int64_t expert_stride, int act, void* y, void* stream) {
  LM_CHECK_ARG(h && w_up && y && n > 0 && top > 0 && width > 0 && ff > 0 && n * top <= 65535 && act == 0);
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return AO_B200_ERR_UNSUPPORTED;
  dim3 grid((unsigned)((ff + kWarps - 1) / kWarps), (unsigned)(n * top));
  LM_DISPATCH(dt, {
    auto kern = expert_up_act_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    kern<<<grid, kWarps * 32, smem, lm_stream(stream)>>>(static_cast<const T*>(h), static_cast<const T*>(w_up), idx, top, width, ff,
                                                        expert_stride, act, static_cast<T*>(y));
  });
  return lm_launch_status();
}

extern "C" int ao_lm_gather_rows(const void* h, int dt, const int64_t* src, int top, int64_t m, int64_t width, void* xs,
                                 void* stream) {
  LM_CHECK_ARG(h && src && xs && top > 0 && m > 0 && width > 0);
  LM_DISPATCH(dt, gather_rows_kernel<T><<<(unsigned)m, 256, 0, lm_stream(stream)>>>(static_cast<const T*>(h), src, top, width,
                                                                                    static_cast<T*>(xs)));
  return lm_launch_status();
}

extern "C" int ao_lm_scatter_add_rows(const void* y, int dt, const int64_t* src, const float* weight, int top, int64_t m,
                                      int64_t width, float* out, void* stream) {
  LM_CHECK_ARG(y && src && weight && out && top > 0 && m > 0 && width > 0);
  LM_DISPATCH(dt, scatter_add_rows_kernel<T><<<(unsigned)m, 256, 0, lm_stream(stream)>>>(static_cast<const T*>(y), src, weight,
                                                                                         top, width, out));
  return lm_launch_status();
}
