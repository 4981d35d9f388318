// Row kernels of designs whose norm is a layer norm (mean and variance, weight and bias) on an fp32 residual that grows by
// a constant times each sublayer's result: the residual add fused with the next sublayer's norm; rotary positions applied
// in place to an fp32 projection (both pairings of coordinates); the inputs of a time-mixing layer that blends every row
// with its predecessor through several learned vectors at once; element-wise activations between two projections.
#include "lm_common.cuh"

using namespace lm;

namespace {

// x[r] += mult * y[r];  out[i] = (x[r] - mean) / sqrt(var + eps) * w + b,  r = rows ? rows[i] : i.  One CTA per row; the row
// stays in shared memory between the statistics and the output (out_f32 may be x itself: a norm in place).
template <typename T>
__global__ void add_layer_norm_kernel(float* x, const float* __restrict__ y, float mult,
                                      const int32_t* __restrict__ rows, int64_t W, const T* __restrict__ weight,
                                      const T* __restrict__ bias, float eps, float* out_f32, T* __restrict__ out) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  const int64_t i = blockIdx.x, r = rows ? (int64_t)rows[i] : i;
  float* xr = x + r * W;
  float s = 0.f;
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) {
    float v = xr[w];
    if (y) {
      v = fmaf(mult, y[r * W + w], v);
      xr[w] = v;
    }
    row[w] = v;
    s += v;
  }
  if (!weight) return;
  const float mean = block_sum(s, scratch) / (float)W;
  float ss = 0.f;
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) {
    const float d = row[w] - mean;
    ss = fmaf(d, d, ss);
  }
  const float k = 1.f / sqrtf(block_sum(ss, scratch) / (float)W + eps);
  for (int64_t w = threadIdx.x; w < W; w += blockDim.x) {
    const float v = (row[w] - mean) * k * ldf(weight + w) + (bias ? ldf(bias + w) : 0.f);
    if (out_f32) out_f32[i * W + w] = v;
    if (out) stf(out + i * W + w, v);
  }
}

// Rotation of the first rot_dims coordinates of every head of two blocks of an fp32 row (queries and keys), in place, then a
// constant factor per block.  pairing 0: (2i, 2i + 1); pairing 1: (i, i + rot_dims / 2).  angle = pos * inv_freq[i], fp32.
__global__ void rotary_rows_kernel(float* __restrict__ proj, int64_t ld, const int32_t* __restrict__ pos,
                                   const float* __restrict__ inv_freq, int rot_dims, int pairing, int d, int64_t off_a,
                                   int heads_a, float scale_a, int64_t off_b, int heads_b, float scale_b) {
  const int64_t t = blockIdx.x;
  const float p = (float)pos[t];
  const int half = rot_dims / 2, per = d - half;     // work items per head: the pairs, then the coordinates that pass
  float* row = proj + t * ld;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < (heads_a + heads_b) * per; i += gridDim.y * blockDim.x) {
    const int hd = i / per, e = i - hd * per;
    float* hp = hd < heads_a ? row + off_a + (int64_t)hd * d : row + off_b + (int64_t)(hd - heads_a) * d;
    const float sc = hd < heads_a ? scale_a : scale_b;
    if (e < half) {
      const int ia = pairing ? e : 2 * e, ib = pairing ? e + half : 2 * e + 1;
      float sn, cs;
      sincosf(p * inv_freq[e], &sn, &cs);
      const float u = hp[ia], v = hp[ib];
      hp[ia] = (u * cs - v * sn) * sc;
      hp[ib] = (v * cs + u * sn) * sc;
    } else if (sc != 1.f) {
      hp[rot_dims + (e - half)] *= sc;
    }
  }
}

// mixes[s][t][:] = h[t] + (prev - h[t]) * mu[s][:], s < n_mix; prev = h[t - 1] inside a segment, the slot's saved row when
// the segment continues an earlier step, zeros at position 0.
template <typename T>
__global__ void token_shift_mix_kernel(const float* __restrict__ h, const T* __restrict__ mu, int n_mix,
                                       const float* __restrict__ state, const int32_t* __restrict__ slot,
                                       const int32_t* __restrict__ pos, const int32_t* __restrict__ back, int64_t n, int64_t W,
                                       T* __restrict__ mixes) {
  const int64_t t = blockIdx.x;
  const float* prev = nullptr;
  if (pos[t] > 0) prev = back[t] > 0 ? h + (t - 1) * W : state + (int64_t)slot[t] * W;
  for (int64_t w = blockIdx.y * blockDim.x + threadIdx.x; w < W; w += (int64_t)gridDim.y * blockDim.x) {
    const float v = h[t * W + w];
    const float dlt = (prev ? prev[w] : 0.f) - v;
    for (int s = 0; s < n_mix; ++s) stf(mixes + ((int64_t)s * n + t) * W + w, fmaf(dlt, ldf(mu + (int64_t)s * W + w), v));
  }
}

template <typename TI, typename TO>
__global__ void unary_rows_kernel(const TI* in, int64_t cols, int kind, float param, const float* __restrict__ row_scale,
                                  int64_t ld_scale, TO* out) {
  const int64_t t = blockIdx.x;
  const float k = row_scale ? row_scale[t * ld_scale] : 1.f;
  for (int64_t c = blockIdx.y * blockDim.x + threadIdx.x; c < cols; c += (int64_t)gridDim.y * blockDim.x) {
    const float z = ldf(in + t * cols + c);
    float v;
    if (kind == 0) {
      const float r = fmaxf(z, 0.f);
      v = r * r;
    } else if (kind == 1) {
      v = tanhf(z);
    } else {
      v = param * tanhf(z / param);
    }
    stf(out + t * cols + c, v * k);
  }
}

inline unsigned threads_for(int64_t width) { return width >= 1024 ? 256 : 128; }
// threads of a kernel that reduces over its row: four values per thread up to the largest block
inline unsigned reduce_threads_for(int64_t width) {
  const int64_t t = ((width / 4 + 31) / 32) * 32;
  return (unsigned)(t < 128 ? 128 : t > 1024 ? 1024 : t);
}
// CTAs per row of an element-wise kernel: one when many rows fill the GPU, else enough that a thread sees few elements (a
// decoded token's row must not be walked by one CTA)
inline dim3 row_grid(int64_t n, int64_t items, unsigned threads) {
  int64_t parts = 1;
  if (n < 296) {
    parts = (items + 2 * threads - 1) / (2 * threads);
    const int64_t room = (592 + n - 1) / n;
    parts = parts > room ? room : parts < 1 ? 1 : parts;
  }
  return dim3((unsigned)n, (unsigned)parts);
}

}  // namespace

extern "C" int ao_lm_add_layer_norm(float* x, const float* y, float mult, const int32_t* rows, int64_t m, int64_t width,
                                    const void* weight, const void* bias, int dt, float eps, float* out_f32, void* out,
                                    void* stream) {
  LM_CHECK_ARG(x && m > 0 && width > 0 && (weight || y) && (!weight || out_f32 || out) && !(y && rows));
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return AO_B200_ERR_UNSUPPORTED;
  LM_DISPATCH(dt, {
    auto kern = add_layer_norm_kernel<T>;
    if (smem > 48 * 1024) {
      static bool set = false;
      if (!set) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return AO_B200_ERR_CUDA;
        set = true;
      }
    }
    // many rows fill the GPU with small blocks; a few rows (decoded tokens) want the row spread over a large one
    kern<<<(unsigned)m, m < 296 ? reduce_threads_for(width) : threads_for(width), smem, lm_stream(stream)>>>(x, y, mult, rows, width, static_cast<const T*>(weight),
                                                                        static_cast<const T*>(bias), eps, out_f32,
                                                                        static_cast<T*>(out));
  });
  return lm_launch_status();
}

extern "C" int ao_lm_rotary_rows(float* proj, int64_t ld, int64_t n, const int32_t* pos, const float* inv_freq, int rot_dims,
                                 int pairing, int d, int64_t off_a, int heads_a, float scale_a, int64_t off_b, int heads_b,
                                 float scale_b, void* stream) {
  LM_CHECK_ARG(proj && pos && n > 0 && d > 0 && rot_dims >= 0 && rot_dims <= d && rot_dims % 2 == 0 && (rot_dims == 0 || inv_freq));
  LM_CHECK_ARG(heads_a >= 0 && heads_b >= 0 && heads_a + heads_b > 0 && (pairing == 0 || pairing == 1));
  if (rot_dims == 0 && scale_a == 1.f && scale_b == 1.f) return AO_B200_OK;
  rotary_rows_kernel<<<row_grid(n, (int64_t)(heads_a + heads_b) * (d - rot_dims / 2), 128), 128, 0, lm_stream(stream)>>>(
      proj, ld, pos, inv_freq, rot_dims, pairing, d, off_a, heads_a, scale_a, off_b, heads_b, scale_b);
  return lm_launch_status();
}

extern "C" int ao_lm_token_shift_mix(const float* h, const void* mu, int n_mix, int dt, const float* state, const int32_t* slot,
                                     const int32_t* pos, const int32_t* back, int64_t n, int64_t width, void* mixes, void* stream) {
  LM_CHECK_ARG(h && mu && state && slot && pos && back && mixes && n > 0 && width > 0 && n_mix > 0 && n_mix <= 16);
  LM_DISPATCH(dt, token_shift_mix_kernel<T><<<row_grid(n, width, threads_for(width)), threads_for(width), 0, lm_stream(stream)>>>(
                      h, static_cast<const T*>(mu), n_mix, state, slot, pos, back, n, width, static_cast<T*>(mixes)));
  return lm_launch_status();
}

extern "C" int ao_lm_unary_rows(const void* in, int in_dt, int64_t n, int64_t cols, int kind, float param, const float* row_scale,
                                int64_t ld_scale, void* out, int out_dt, void* stream) {
  LM_CHECK_ARG(in && out && n > 0 && cols > 0 && kind >= 0 && kind <= 2 && (kind != 2 || param > 0.f));
  const cudaStream_t st = lm_stream(stream);
  const unsigned th = threads_for(cols);
  const dim3 grid = row_grid(n, cols, th);
  if (in_dt == AO_LM_F32 && out_dt == AO_LM_F32)
    unary_rows_kernel<float, float><<<grid, th, 0, st>>>(static_cast<const float*>(in), cols, kind, param, row_scale, ld_scale,
                                                                static_cast<float*>(out));
  else if (in_dt == AO_LM_F32 && out_dt == AO_LM_BF16)
    unary_rows_kernel<float, __nv_bfloat16><<<grid, th, 0, st>>>(static_cast<const float*>(in), cols, kind, param, row_scale,
                                                                        ld_scale, static_cast<__nv_bfloat16*>(out));
  else if (in_dt == AO_LM_BF16 && out_dt == AO_LM_BF16)
    unary_rows_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, th, 0, st>>>(static_cast<const __nv_bfloat16*>(in), cols, kind,
                                                                                param, row_scale, ld_scale,
                                                                                static_cast<__nv_bfloat16*>(out));
  else
    return AO_B200_ERR_INVALID_ARG;
  return lm_launch_status();
}
