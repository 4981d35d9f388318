// Row-wise kernels of the fp32 residual stream: embedding gather, token shift, residual add with a scalar-weight RMS
// norm (+ token-shift memory, + depth-weighted average of the layer results, + storage-type copy), latent-attention
// projection split (latent norm, rotary, gate), clipped-GLU activation, greedy argmax.  One CTA per token row.
#include "lm_common.cuh"

using namespace lm;

namespace {

constexpr int kRowThreads = 256;
// threads of a row's CTA: a step of few rows has few CTAs, so each row is spread over more threads (more loads in flight)
inline unsigned row_threads(int64_t rows, int64_t width) {
  if (rows >= 128) return kRowThreads;
  unsigned t = kRowThreads;
  while (t < 1024 && (int64_t)t * 4 < width) t *= 2;
  return t;
}

template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int64_t* __restrict__ tok, int64_t W, float* __restrict__ x) {
  const int64_t t = blockIdx.x;
  const T* row = table + tok[t] * W;
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) x[t * W + w] = ldf(row + w);
}

template <typename T>
__global__ void token_shift_kernel(const float* __restrict__ x, const T* __restrict__ mu, const float* __restrict__ state,
                                   const int32_t* __restrict__ slot, const int32_t* __restrict__ pos, int64_t W,
                                   T* __restrict__ h) {
  const int64_t t = blockIdx.x;
  const int p = pos[t], s = slot[t];
  const float* prev = nullptr;
  if (p > 0) prev = (t > 0 && slot[t - 1] == s && pos[t - 1] == p - 1) ? x + (t - 1) * W : state + (int64_t)s * W;
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) {
    const float v = x[t * W + w];
    const float pv = prev ? prev[w] : 0.f;
    stf(h + t * W + w, v + (pv - v) * ldf(mu + w));
  }
}

template <typename T, typename TY>
__global__ void residual_norm_kernel(const float* __restrict__ x_in, const TY* __restrict__ y, const T* __restrict__ g,
                                     float mult, float eps, int64_t n, int64_t W, float* __restrict__ x_out,
                                     float* __restrict__ state, const int32_t* __restrict__ slot,
                                     const float* __restrict__ streams, int n_streams, int64_t stream_stride,
                                     const T* __restrict__ coef, float* __restrict__ avg_out, T* __restrict__ cast_out) {
  __shared__ float scratch[33];
  const int64_t t = blockIdx.x;
  const TY* yr = y + t * W;
  float ss = 0.f;
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) {
    const float v = ldf(yr + w);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float k = mult * ldf(g) / sqrtf(ss / (float)W + eps);
  const bool save = state && (t == n - 1 || slot[t + 1] != slot[t]);
  float* st = save ? state + (int64_t)slot[t] * W : nullptr;
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) {
    const float xi = x_in[t * W + w];
    if (st) st[w] = xi;
    float v = fmaf(k, ldf(yr + w), xi);
    x_out[t * W + w] = v;
    if (streams) {
      float a = ldf(coef + n_streams) * v;
      for (int j = n_streams - 1; j >= 0; --j) a = fmaf(ldf(coef + j), streams[j * stream_stride + t * W + w], a);
      avg_out[t * W + w] = a;
      v = a;
    }
    if (cast_out) stf(cast_out + t * W + w, v);
  }
}

template <typename T>
__global__ void scalar_norm_rows_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, int64_t W,
                                        const T* __restrict__ g, float eps, T* __restrict__ out) {
  __shared__ float scratch[33];
  const int64_t i = blockIdx.x;
  const float* xr = x + (rows ? (int64_t)rows[i] : i) * W;
  float ss = 0.f;
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) ss = fmaf(xr[w], xr[w], ss);
  ss = block_sum(ss, scratch);
  const float k = ldf(g) / sqrtf(ss / (float)W + eps);
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) stf(out + i * W + w, xr[w] * k);
}

template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ proj, int64_t ld, int64_t n, int H, int dn, int dr, int R,
                                   int64_t q_off, int64_t kv_off, int64_t g_off, const T* __restrict__ c_norm, float eps,
                                   int rot_dims, const float* __restrict__ inv_freq, const int32_t* __restrict__ slot,
                                   const int32_t* __restrict__ pos, T* __restrict__ c_cache, T* __restrict__ kr_cache,
                                   int64_t S, T* __restrict__ qn, float* __restrict__ qr, float* __restrict__ gate) {
  __shared__ float scratch[33];
  const int64_t t = blockIdx.x;
  const T* row = proj + t * ld;
  const int p = pos[t];
  const float fp = (float)p;
  const int half = rot_dims / 2;
  // unrotated query parts, head-major
  for (int i = threadIdx.x; i < H * dn; i += blockDim.x) {
    const int h = i / dn, d = i - h * dn;
    qn[((int64_t)h * n + t) * dn + d] = row[q_off + (int64_t)h * (dn + dr) + d];
  }
  // rotated query parts: one thread per pair, then the tail that is not rotated
  for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
    const int h = i / half, j = i - h * half;
    const T* q = row + q_off + (int64_t)h * (dn + dr) + dn;
    float sn, cs;
    sincosf(fp * inv_freq[j], &sn, &cs);
    const float u = ldf(q + 2 * j), v = ldf(q + 2 * j + 1);
    float* o = qr + (t * H + h) * dr;
    o[2 * j] = u * cs - v * sn;
    o[2 * j + 1] = v * cs + u * sn;
  }
  for (int i = threadIdx.x; i < H * (dr - 2 * half); i += blockDim.x) {
    const int h = i / (dr - 2 * half), d = 2 * half + (i - h * (dr - 2 * half));
    qr[(t * H + h) * dr + d] = ldf(row + q_off + (int64_t)h * (dn + dr) + dn + d);
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) gate[t * H + h] = 1.f / (1.f + expf(-ldf(row + g_off + h)));
  if (kv_off < 0) return;   // uniform over the block
  const T* kv = row + kv_off;
  const int64_t at = (int64_t)slot[t] * S + p;
  float ss = 0.f;
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const float v = ldf(kv + i);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float k = 1.f / sqrtf(ss / (float)R + eps);
  for (int i = threadIdx.x; i < R; i += blockDim.x) stf(c_cache + at * R + i, ldf(kv + i) * k * ldf(c_norm + i));
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float sn, cs;
    sincosf(fp * inv_freq[j], &sn, &cs);
    const float u = ldf(kv + R + 2 * j), v = ldf(kv + R + 2 * j + 1);
    stf(kr_cache + at * dr + 2 * j, u * cs - v * sn);
    stf(kr_cache + at * dr + 2 * j + 1, v * cs + u * sn);
  }
  for (int d = 2 * half + threadIdx.x; d < dr; d += blockDim.x) kr_cache[at * dr + d] = kv[R + d];
}

// A sublayer's result enters the residual through its own RMS norm (a weight per coordinate), and the next sublayer's
// input norm is taken in the same pass over the row:
//   y += y_bias (a projection's bias that its GEMM left out);
//   x += y / sqrt(mean(y^2) + eps) * post_w;   x += add_rows[t];   x += add_vec;   h = x / sqrt(mean(x^2) + eps) * next_w.
// Every part but x is optional.  The row stays in registers between the two norms (up to kPostPer values per thread).
constexpr int kPostPer = 8;
template <typename T, typename TY, bool BIAS>
__global__ void __launch_bounds__(1024) postnorm_residual_kernel(float* __restrict__ x, const TY* __restrict__ y,
                                                                 const float* __restrict__ y_bias, const T* __restrict__ post_w,
                                                                 const float* __restrict__ add_rows,
                                                                 const T* __restrict__ add_vec, const T* __restrict__ next_w,
                                                                 float eps, int64_t W, T* __restrict__ h) {
  __shared__ float scratch[33];
  const int64_t t = blockIdx.x;
  float* xr = x + t * W;
  const bool in_regs = W <= (int64_t)kPostPer * blockDim.x;
  float keep[kPostPer];      // the sublayer's result first, the new residual afterwards
  float xk[kPostPer];        // the residual's old values: in flight while the result's norm is reduced
#pragma unroll
  for (int i = 0; i < kPostPer; ++i) {
    const int64_t w = threadIdx.x + (int64_t)i * blockDim.x;
    xk[i] = w < W ? xr[w] : 0.f;
  }
  float k = 0.f;
  if (y) {
    const TY* yr = y + t * W;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kPostPer; ++i) {
      const int64_t w = threadIdx.x + (int64_t)i * blockDim.x;
      keep[i] = w < W ? ldf(yr + w) + (BIAS ? y_bias[w] : 0.f) : 0.f;
      ss = fmaf(keep[i], keep[i], ss);
    }
    for (int64_t w = threadIdx.x + (int64_t)kPostPer * blockDim.x; w < W; w += blockDim.x) {
      const float v = ldf(yr + w) + (BIAS ? y_bias[w] : 0.f);
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    k = 1.f / sqrtf(ss / (float)W + eps);
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kPostPer; ++i) {
    const int64_t w = threadIdx.x + (int64_t)i * blockDim.x;
    if (w < W) {
      float v = xk[i];
      if (y) v = fmaf(keep[i] * k, post_w ? ldf(post_w + w) : 1.f, v);
      if (add_rows) v += add_rows[t * W + w];
      if (add_vec) v += ldf(add_vec + w);
      xr[w] = v;
      keep[i] = v;
      ss = fmaf(v, v, ss);
    }
  }
  for (int64_t w = threadIdx.x + (int64_t)kPostPer * blockDim.x; w < W; w += blockDim.x) {
    float v = xr[w];
    if (y) v = fmaf((ldf(y + t * W + w) + (BIAS ? y_bias[w] : 0.f)) * k, post_w ? ldf(post_w + w) : 1.f, v);
    if (add_rows) v += add_rows[t * W + w];
    if (add_vec) v += ldf(add_vec + w);
    xr[w] = v;
    ss = fmaf(v, v, ss);
  }
  if (!next_w) return;
  ss = block_sum(ss, scratch);
  const float kn = 1.f / sqrtf(ss / (float)W + eps);
  if (in_regs) {
#pragma unroll
    for (int i = 0; i < kPostPer; ++i) {
      const int64_t w = threadIdx.x + (int64_t)i * blockDim.x;
      if (w < W) stf(h + t * W + w, keep[i] * kn * ldf(next_w + w));
    }
  } else {
    for (int64_t w = threadIdx.x; w < W; w += blockDim.x) stf(h + t * W + w, xr[w] * kn * ldf(next_w + w));
  }
}

template <typename T>
__global__ void glu_act_kernel(const T* __restrict__ gu, int64_t n, int64_t ff, float limit, float alpha, float shift,
                               T* __restrict__ y) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * ff) return;
  const int64_t t = i / ff, f = i - t * ff;
  const float g = fminf(ldf(gu + t * 2 * ff + f), limit);
  const float u = fminf(fmaxf(ldf(gu + t * 2 * ff + ff + f), -limit), limit);
  stf(y + i, g / (1.f + expf(-alpha * g)) * (u + shift));
}

// bf16 rows with ff a multiple of 8: one thread makes 8 outputs from two 16-byte loads
__global__ void glu_act_vec_kernel(const __nv_bfloat16* __restrict__ gu, int64_t n, int64_t ff, float limit, float alpha,
                                   float shift, __nv_bfloat16* __restrict__ y) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, per = ff / 8;
  if (i >= n * per) return;
  const int64_t t = i / per, f = (i - t * per) * 8;
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(gu + t * 2 * ff + f));
  const uint4 b = __ldg(reinterpret_cast<const uint4*>(gu + t * 2 * ff + ff + f));
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float r[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const float gv = fminf(__uint_as_float(e ? aw[j] & 0xFFFF0000u : aw[j] << 16), limit);
      const float uv = fminf(fmaxf(__uint_as_float(e ? bw[j] & 0xFFFF0000u : bw[j] << 16), -limit), limit);
      r[e] = gv / (1.f + expf(-alpha * gv)) * (uv + shift);
    }
    const __nv_bfloat162 pk = __floats2bfloat162_rn(r[0], r[1]);
    o[j] = *reinterpret_cast<const uint32_t*>(&pk);
  }
  *reinterpret_cast<uint4*>(y + t * ff + f) = make_uint4(o[0], o[1], o[2], o[3]);
}

template <typename T>
__global__ void add_cast_kernel(const T* __restrict__ b, int64_t count, float* __restrict__ a) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) a[i] += ldf(b + i);
}

__global__ void argmax_kernel(const float* __restrict__ logits, int64_t ld, int64_t V, int64_t* __restrict__ out) {
  __shared__ float bv[32];
  __shared__ int64_t bi[32];
  const float* row = logits + blockIdx.x * ld;
  float best = -INFINITY;
  int64_t at = V;
  int64_t i = threadIdx.x;
  for (; i + 3 * (int64_t)blockDim.x < V; i += 4 * (int64_t)blockDim.x) {   // four loads in flight per thread
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = row[i + j * (int64_t)blockDim.x];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (v[j] > best) best = v[j], at = i + j * (int64_t)blockDim.x;     // ascending indices: the first of equals stays
  }
  for (; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best) best = v, at = i;
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, at, o);
    if (ov > best || (ov == best && oi < at)) best = ov, at = oi;
  }
  if ((threadIdx.x & 31) == 0) bv[threadIdx.x >> 5] = best, bi[threadIdx.x >> 5] = at;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (bv[w] > best || (bv[w] == best && bi[w] < at)) best = bv[w], at = bi[w];
    out[blockIdx.x] = at < V ? at : 0;
  }
}

}  // namespace

int g_lm_last_cuda_error = 0;

extern "C" const char* ao_lm_last_cuda_error(void) {
  return g_lm_last_cuda_error ? cudaGetErrorString((cudaError_t)g_lm_last_cuda_error) : "";
}

extern "C" int ao_lm_abi_version(void) { return 1; }

extern "C" int ao_lm_embed(const void* table, int dt, const int64_t* tok, int64_t n, int64_t width, float* x, void* stream) {
  LM_CHECK_ARG(table && tok && x && n > 0 && width > 0);
  LM_DISPATCH(dt, embed_kernel<T><<<(unsigned)n, row_threads(n, width), 0, lm_stream(stream)>>>(static_cast<const T*>(table), tok, width, x));
  return lm_launch_status();
}

extern "C" int ao_lm_token_shift(const float* x, const void* mu, int dt, const float* state, const int32_t* slot,
                                 const int32_t* pos, int64_t n, int64_t width, void* h, void* stream) {
  LM_CHECK_ARG(x && mu && state && slot && pos && h && n > 0 && width > 0);
  LM_DISPATCH(dt, token_shift_kernel<T><<<(unsigned)n, row_threads(n, width), 0, lm_stream(stream)>>>(
                      x, static_cast<const T*>(mu), state, slot, pos, width, static_cast<T*>(h)));
  return lm_launch_status();
}

extern "C" int ao_lm_residual_norm(const float* x_in, const void* y, int y_dt, const void* g, int dt, float mult, float eps,
                                   int64_t n, int64_t width, float* x_out, float* state, const int32_t* slot,
                                   const float* streams, int n_streams, int64_t stream_stride, const void* coef,
                                   float* avg_out, void* cast_out, void* stream) {
  LM_CHECK_ARG(x_in && y && g && x_out && n > 0 && width > 0);
  LM_CHECK_ARG((!state || slot) && (!streams || (coef && avg_out && n_streams >= 0)));
  LM_DISPATCH(dt, {
    if (y_dt == AO_LM_F32)
      residual_norm_kernel<T, float><<<(unsigned)n, row_threads(n, width), 0, lm_stream(stream)>>>(
          x_in, static_cast<const float*>(y), static_cast<const T*>(g), mult, eps, n, width, x_out, state, slot, streams,
          n_streams, stream_stride, static_cast<const T*>(coef), avg_out, static_cast<T*>(cast_out));
    else if (y_dt == dt)
      residual_norm_kernel<T, T><<<(unsigned)n, row_threads(n, width), 0, lm_stream(stream)>>>(
          x_in, static_cast<const T*>(y), static_cast<const T*>(g), mult, eps, n, width, x_out, state, slot, streams,
          n_streams, stream_stride, static_cast<const T*>(coef), avg_out, static_cast<T*>(cast_out));
    else
      return AO_B200_ERR_INVALID_ARG;
  });
  return lm_launch_status();
}

extern "C" int ao_lm_scalar_norm_rows(const float* x, const int32_t* rows, int64_t m, int64_t width, const void* g, int dt,
                                      float eps, void* out, void* stream) {
  LM_CHECK_ARG(x && g && out && m > 0 && width > 0);
  LM_DISPATCH(dt, scalar_norm_rows_kernel<T><<<(unsigned)m, row_threads(m, width), 0, lm_stream(stream)>>>(
                      x, rows, width, static_cast<const T*>(g), eps, static_cast<T*>(out)));
  return lm_launch_status();
}

extern "C" int ao_lm_latent_prep(const void* proj, int dt, int64_t ld, int64_t n, int H, int dn, int dr, int R, int64_t q_off,
                                 int64_t kv_off, int64_t g_off, const void* c_norm, float eps, int rot_dims,
                                 const float* inv_freq, const int32_t* slot, const int32_t* pos, void* c_cache,
                                 void* kr_cache, int64_t S, void* qn, float* qr, float* gate, void* stream) {
  LM_CHECK_ARG(proj && slot && pos && qn && qr && gate && n > 0 && H > 0 && dn >= 0 && dr >= 0 && R > 0);
  LM_CHECK_ARG(rot_dims >= 0 && rot_dims <= dr && rot_dims % 2 == 0 && (rot_dims == 0 || inv_freq));
  LM_CHECK_ARG(kv_off < 0 || (c_norm && c_cache && kr_cache && S > 0));
  LM_DISPATCH(dt, latent_prep_kernel<T><<<(unsigned)n, row_threads(n, (int64_t)H * (dn + dr)), 0, lm_stream(stream)>>>(
                      static_cast<const T*>(proj), ld, n, H, dn, dr, R, q_off, kv_off, g_off, static_cast<const T*>(c_norm), eps,
                      rot_dims, inv_freq, slot, pos, static_cast<T*>(c_cache), static_cast<T*>(kr_cache), S,
                      static_cast<T*>(qn), qr, gate));
  return lm_launch_status();
}

extern "C" int ao_lm_glu_act_shift(const void* gu, int dt, int64_t n, int64_t ff, float limit, float alpha, float shift, void* y,
                                   void* stream) {
  LM_CHECK_ARG(gu && y && n > 0 && ff > 0);
  if (dt == AO_LM_BF16 && ff % 8 == 0 && reinterpret_cast<uintptr_t>(gu) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0) {
    glu_act_vec_kernel<<<(unsigned)((n * (ff / 8) + 255) / 256), 256, 0, lm_stream(stream)>>>(
        static_cast<const __nv_bfloat16*>(gu), n, ff, limit, alpha, shift, static_cast<__nv_bfloat16*>(y));
    return lm_launch_status();
  }
  const unsigned grid = (unsigned)((n * ff + 255) / 256);
  LM_DISPATCH(dt, glu_act_kernel<T><<<grid, 256, 0, lm_stream(stream)>>>(static_cast<const T*>(gu), n, ff, limit, alpha, shift,
                                                                         static_cast<T*>(y)));
  return lm_launch_status();
}

extern "C" int ao_lm_glu_act(const void* gu, int dt, int64_t n, int64_t ff, float limit, float alpha, void* y, void* stream) {
  return ao_lm_glu_act_shift(gu, dt, n, ff, limit, alpha, 1.f, y, stream);
}

namespace {
template <typename T, typename TY, bool BIAS>
void launch_postnorm(float* x, const void* y, const float* y_bias, const void* post_w, const float* add_rows, const void* add_vec,
                     const void* next_w, float eps, int64_t n, int64_t width, void* h, unsigned threads, void* stream) {
  postnorm_residual_kernel<T, TY, BIAS><<<(unsigned)n, threads, 0, lm_stream(stream)>>>(
      x, static_cast<const TY*>(y), y_bias, static_cast<const T*>(post_w), add_rows, static_cast<const T*>(add_vec),
      static_cast<const T*>(next_w), eps, width, static_cast<T*>(h));
}
}  // namespace

extern "C" int ao_lm_postnorm_residual(float* x, const void* y, int y_dt, const float* y_bias, const void* post_w, const float* add_rows,
                                       const void* add_vec, const void* next_w, int dt, float eps, int64_t n, int64_t width,
                                       void* h, void* stream) {
  LM_CHECK_ARG(x && n > 0 && width > 0 && (!next_w || h) && (y || !y_bias) && (y_dt == AO_LM_BF16 || y_dt == AO_LM_F32));
  unsigned threads = row_threads(n, width);
  while (threads < 1024 && (int64_t)threads * kPostPer < width) threads *= 2;   // the row stays in registers up to 8192 values
  LM_DISPATCH(dt, {
if (y_dt == AO_LM_F32) {
      if (y_bias) launch_postnorm<T, float, true>(x, y, y_bias, post_w, add_rows, add_vec, next_w, eps, n, width, h, threads, stream);
      else launch_postnorm<T, float, false>(x, y, y_bias, post_w, add_rows, add_vec, next_w, eps, n, width, h, threads, stream);
    } else {
      if (y_bias) launch_postnorm<T, __nv_bfloat16, true>(x, y, y_bias, post_w, add_rows, add_vec, next_w, eps, n, width, h, threads, stream);
      else launch_postnorm<T, __nv_bfloat16, false>(x, y, y_bias, post_w, add_rows, add_vec, next_w, eps, n, width, h, threads, stream);
    }
  });
  return lm_launch_status();
}

extern "C" int ao_lm_add_cast(const void* b, int dt, int64_t count, float* a_inout, void* stream) {
  LM_CHECK_ARG(b && a_inout && count > 0);
  const unsigned grid = (unsigned)((count + 255) / 256);
  LM_DISPATCH(dt, add_cast_kernel<T><<<grid, 256, 0, lm_stream(stream)>>>(static_cast<const T*>(b), count, a_inout));
  return lm_launch_status();
}

extern "C" int ao_lm_argmax(const float* logits, int64_t ld, int64_t B, int64_t V, int64_t* out, void* stream) {
  LM_CHECK_ARG(logits && out && B > 0 && V > 0 && ld >= V);
  argmax_kernel<<<(unsigned)B, 1024, 0, lm_stream(stream)>>>(logits, ld, V, out);
  return lm_launch_status();
}
