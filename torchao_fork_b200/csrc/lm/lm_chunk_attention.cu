// Attention whose mask is cut into chunks of C positions counted from the start of the sequence: a query sees the keys
// of its own chunk up to itself.  Grouped heads (H query heads over G key/value heads), queries and keys divided by
// their root mean square per head, score = softcap * tanh(scale * q.k / softcap) + bias[distance][head], ordinary
// softmax, and the result multiplied coordinate by coordinate with sigmoid(gate).
//
// Only the current chunk of a sequence is ever read again, so the cache is a ring of C rows per sequence slot:
// position p lives in row p % C.  A step's own keys and values are read from the step's buffers and appended to the ring
// AFTER the attention (a long prompt portion would otherwise overwrite rows that its first chunk still needs):
//     ao_lm_qk_prep -> ao_lm_chunk_attention -> ao_lm_ring_append.
// Key index kk of a tile = position (chunk start + kk); the first n_ring of them come from the ring, the rest from the
// step's rows.  Scores, weights, norms and the gate are fp32 in both storage types.
#include "lm_common.cuh"

using namespace lm;

namespace {

constexpr int kWarps = 8;
constexpr int kKeys = 32;            // keys per shared-memory block
constexpr int kPairSlots = 4;        // (row, query head) pairs per warp
constexpr int kMaxDvLane = 8;        // value size <= 32 * kMaxDvLane

// q: unit RMS per head -> fp32 [n][H][d];  k: unit RMS per head -> storage type [n][G][d];  v -> storage type [n][G][dv]
template <typename T>
__global__ void qk_prep_kernel(const float* __restrict__ proj, int64_t ld, int64_t q_off, int64_t k_off, int64_t v_off, int H,
                               int G, int d, int dv, float eps, float* __restrict__ qn, T* __restrict__ kn, T* __restrict__ vn) {
  const int64_t t = blockIdx.x;
  const float* row = proj + t * ld;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int h = warp; h < H + G; h += nw) {
    const float* src = h < H ? row + q_off + (int64_t)h * d : row + k_off + (int64_t)(h - H) * d;
    float ss = 0.f;
    for (int c = lane; c < d; c += 32) ss = fmaf(src[c], src[c], ss);
    ss = warp_sum(ss);
    const float k = 1.f / sqrtf(ss / (float)d + eps);
    if (h < H) {
      float* dst = qn + (t * H + h) * d;
      for (int c = lane; c < d; c += 32) dst[c] = src[c] * k;
    } else {
      T* dst = kn + (t * G + (h - H)) * d;
      for (int c = lane; c < d; c += 32) stf(dst + c, src[c] * k);
    }
  }
  for (int c = threadIdx.x; c < G * dv; c += blockDim.x) stf(vn + t * G * dv + c, row[v_off + c]);
}

// The same split with what a design may put between the projection and the attention: biases added to the projection,
// a learned weight per coordinate on the unit-RMS queries and keys (shared by all heads), and a query temperature that
// grows with the position: q *= 1 + coef * ln(floor((pos + 1) / every) + 1).
template <typename T>
__global__ void qk_norm_prep_kernel(const float* __restrict__ proj, int64_t ld, int64_t q_off, int64_t k_off, int64_t v_off,
                                    const T* __restrict__ q_bias, const T* __restrict__ k_bias, const T* __restrict__ v_bias,
                                    const T* __restrict__ q_weight, const T* __restrict__ k_weight, float temp_coef,
                                    int temp_every, const int32_t* __restrict__ pos, const int32_t* __restrict__ slot,
                                    T* __restrict__ ring_k, T* __restrict__ ring_v, int ring, int H, int G, int d, int dv,
                                    float eps, float* __restrict__ qn, T* __restrict__ kn, T* __restrict__ vn) {
  const int64_t t = blockIdx.x;
  const int64_t rrow = ring_k ? (int64_t)slot[t] * ring + pos[t] : 0;     // the row's place in a cache that never wraps
  const float* row = proj + t * ld;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  float temp = 1.f;
  if (temp_coef != 0.f) temp = 1.f + temp_coef * logf((float)((pos[t] + 1) / temp_every) + 1.f);
  for (int h = warp; h < H + G; h += nw) {
    const bool is_q = h < H;
    const int64_t off = is_q ? (int64_t)h * d : (int64_t)(h - H) * d;
    const float* src = row + (is_q ? q_off : k_off) + off;
    const T* bias = is_q ? q_bias : k_bias;
    const T* wt = is_q ? q_weight : k_weight;
    float ss = 0.f;
    for (int c = lane; c < d; c += 32) {
      const float v = src[c] + (bias ? ldf(bias + off + c) : 0.f);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float k = (is_q ? temp : 1.f) / sqrtf(ss / (float)d + eps);
    for (int c = lane; c < d; c += 32) {
      const float v = (src[c] + (bias ? ldf(bias + off + c) : 0.f)) * k * (wt ? ldf(wt + c) : 1.f);
      if (is_q)
        qn[(t * H + h) * d + c] = v;
      else {
        stf(kn + (t * G + (h - H)) * d + c, v);
        if (ring_k) stf(ring_k + (rrow * G + (h - H)) * d + c, v);
      }
    }
  }
  for (int c = threadIdx.x; c < G * dv; c += blockDim.x) {
    const float v = row[v_off + c] + (v_bias ? ldf(v_bias + c) : 0.f);
    stf(vn + t * G * dv + c, v);
    if (ring_v) stf(ring_v + rrow * G * dv + c, v);
  }
}

template <typename T>
__global__ void ring_append_kernel(const T* __restrict__ kn, const T* __restrict__ vn, int64_t krow, int64_t vrow, int C,
                                   const int32_t* __restrict__ slot, const int32_t* __restrict__ pos,
                                   const int32_t* __restrict__ ahead, T* __restrict__ ring_k, T* __restrict__ ring_v) {
  const int64_t t = blockIdx.x;
  if (ahead[t] >= C) return;   // a later row of the same step takes this ring row
  const int64_t r = (int64_t)slot[t] * C + pos[t] % C;
  for (int64_t c = threadIdx.x; c < krow; c += blockDim.x) ring_k[r * krow + c] = kn[t * krow + c];
  for (int64_t c = threadIdx.x; c < vrow; c += blockDim.x) ring_v[r * vrow + c] = vn[t * vrow + c];
}

struct ChunkArgs {
  const float* qn;           // [n][H][d]
  const void *kn, *vn;       // step rows [n][G][d], [n][G][dv]
  const void *ring_k, *ring_v;
  const float* gate;         // pre-activation, row stride ld_gate, H * dv per row; null: no gate
  int64_t ld_gate;
  const float* bias;         // [H][n_dist]; null: none
  int n_dist;
  const float* sink;         // [H]: exp(sink) joins every row's denominator; null: none
  const int32_t *slot, *pos, *back, *tile_first, *tile_count;
  int H, G, d, dv, C;
  float scale, softcap, out_scale;
  void* out;                 // [n][ld_out], H * dv per row
  int64_t ld_out;
  int n_split;               // > 1: blockIdx.z takes a share of the key blocks and leaves (max, denominator, sums) in ws
  float* ws;                 // [tiles][G][n_split][kWarps * kPairSlots][dv + 2]
};

// One CTA = a tile of consecutive rows of one sequence inside one chunk x one key/value head; a warp owns up to
// kPairSlots (row, query head) pairs and keeps their running maximum, denominator and output in registers.
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) chunk_attention_kernel(ChunkArgs a) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, g = blockIdx.y;
  const int d = a.d, dv = a.dv, C = a.C, rep = a.H / a.G;
  const int first = a.tile_first[tile], count = a.tile_count[tile];
  const int pos0 = a.pos[first], back0 = a.back[first];
  const int off0 = pos0 % C;                       // the first row's place in its chunk
  const int n_ring = max(0, off0 - back0);         // keys of the chunk that earlier steps left in the ring
  const int64_t step_row0 = first - min(back0, off0);
  const int nk = off0 + count;
  const int npairs = count * rep;
  const int KP = d + 1;
  float* Qs = sm;                                  // [npairs][d]
  float* Ks = Qs + (size_t)kWarps * kPairSlots * d;   // [kKeys][d + 1]
  float* Vs = Ks + (size_t)kKeys * KP;             // [kKeys][dv]
  float* Ps = Vs + (size_t)kKeys * dv;             // [kWarps][kKeys]
  const T* ring_k = static_cast<const T*>(a.ring_k) + ((int64_t)a.slot[first] * C * a.G + g) * d;
  const T* ring_v = static_cast<const T*>(a.ring_v) + ((int64_t)a.slot[first] * C * a.G + g) * dv;
  const T* step_k = static_cast<const T*>(a.kn) + (step_row0 * a.G + g) * d;
  const T* step_v = static_cast<const T*>(a.vn) + (step_row0 * a.G + g) * dv;

  for (int i = threadIdx.x; i < npairs * d; i += blockDim.x) {
    const int pr = i / d, c = i - pr * d, r = pr / rep, qh = g * rep + pr % rep;
    Qs[i] = a.qn[((int64_t)(first + r) * a.H + qh) * d + c];
  }
  float mx[kPairSlots], den[kPairSlots], o[kPairSlots][kMaxDvLane];
#pragma unroll
  for (int s = 0; s < kPairSlots; ++s) {
    mx[s] = -INFINITY, den[s] = 0.f;
#pragma unroll
    for (int e = 0; e < kMaxDvLane; ++e) o[s][e] = 0.f;
  }
  // this CTA's share of the key blocks
  const int blocks = (nk + kKeys - 1) / kKeys, per = (blocks + a.n_split - 1) / a.n_split;
  const int k_lo = (int)blockIdx.z * per * kKeys, k_end = min(nk, ((int)blockIdx.z + 1) * per * kKeys);
  for (int k0 = k_lo; k0 < k_end; k0 += kKeys) {
    __syncthreads();   // the previous block is used up (and, the first time, the queries are in place)
    for (int i = threadIdx.x; i < kKeys * d; i += blockDim.x) {
      const int j = i / d, c = i - j * d, kk = k0 + j;
      float v = 0.f;
      if (kk < nk) v = kk < n_ring ? ldf(ring_k + (int64_t)kk * a.G * d + c) : ldf(step_k + (int64_t)(kk - n_ring) * a.G * d + c);
      Ks[j * KP + c] = v;
    }
    for (int i = threadIdx.x; i < kKeys * dv; i += blockDim.x) {
      const int j = i / dv, c = i - j * dv, kk = k0 + j;
      float v = 0.f;
      if (kk < nk) v = kk < n_ring ? ldf(ring_v + (int64_t)kk * a.G * dv + c) : ldf(step_v + (int64_t)(kk - n_ring) * a.G * dv + c);
      Vs[j * dv + c] = v;
    }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < kPairSlots; ++s) {
      const int pr = warp + s * kWarps;
      if (pr >= npairs) continue;                  // uniform over the warp
      const int r = pr / rep, qh = g * rep + pr % rep;
      const int lim = off0 + r;                    // the row's own key index
      if (k0 > lim) continue;
      const float* q = Qs + (size_t)pr * d;
      const float* kr = Ks + (size_t)lane * KP;
      float sc = 0.f;
      for (int c = 0; c < d; ++c) sc = fmaf(q[c], kr[c], sc);
      const int kk = k0 + lane;
      if (kk <= lim) {
        sc *= a.scale;
        if (a.softcap > 0.f) sc = a.softcap * tanhf(sc / a.softcap);
        if (a.bias) sc += a.bias[(int64_t)qh * a.n_dist + min(lim - kk, a.n_dist - 1)];
      } else {
        sc = -INFINITY;
      }
      const float top = fmaxf(mx[s], warp_max(sc));   // key k0 <= lim is visible: top is finite
      const float corr = mx[s] == -INFINITY ? 0.f : expf(mx[s] - top);
      const float p = expf(sc - top);
      mx[s] = top;
      den[s] = den[s] * corr + warp_sum(p);
      Ps[warp * kKeys + lane] = p;
      __syncwarp();
      const float* pw = Ps + warp * kKeys;
#pragma unroll
      for (int e = 0; e < kMaxDvLane; ++e) {
        const int c = lane + 32 * e;
        if (c < dv) {
          float acc = o[s][e] * corr;
          for (int j = 0; j < kKeys; ++j) acc = fmaf(pw[j], Vs[j * dv + c], acc);
          o[s][e] = acc;
        }
      }
      __syncwarp();
    }
  }
  if (a.n_split > 1) {
    // partial results of this share; a share without visible keys leaves max = -inf, denominator 0
#pragma unroll
    for (int s = 0; s < kPairSlots; ++s) {
      const int pr = warp + s * kWarps;
      if (pr >= npairs) continue;
      float* w = a.ws + ((((int64_t)tile * a.G + g) * a.n_split + blockIdx.z) * (kWarps * kPairSlots) + pr) * (dv + 2);
      if (lane == 0) w[0] = mx[s], w[1] = den[s];
#pragma unroll
      for (int e = 0; e < kMaxDvLane; ++e) {
        const int c = lane + 32 * e;
        if (c < dv) w[2 + c] = o[s][e];
      }
    }
    return;
  }
#pragma unroll
  for (int s = 0; s < kPairSlots; ++s) {
    const int pr = warp + s * kWarps;
    if (pr >= npairs) continue;
    const int r = pr / rep, qh = g * rep + pr % rep;
    const int64_t t = first + r;
    const float inv = a.out_scale / (a.sink ? den[s] + expf(a.sink[qh] - mx[s]) : den[s]);
    const float* gt = a.gate ? a.gate + t * a.ld_gate + (int64_t)qh * dv : nullptr;
    T* dst = static_cast<T*>(a.out) + t * a.ld_out + (int64_t)qh * dv;
#pragma unroll
    for (int e = 0; e < kMaxDvLane; ++e) {
      const int c = lane + 32 * e;
      if (c < dv) stf(dst + c, gt ? o[s][e] * inv / (1.f + expf(-gt[c])) : o[s][e] * inv);
    }
  }
}

// the shares of one (tile, key/value head) put together: one warp per (row, query head) pair
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) chunk_attention_merge_kernel(ChunkArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, g = blockIdx.y, dv = a.dv, rep = a.H / a.G;
  const int first = a.tile_first[tile], npairs = a.tile_count[tile] * rep;
  for (int pr = warp; pr < npairs; pr += kWarps) {
    const float* w0 = a.ws + ((((int64_t)tile * a.G + g) * a.n_split) * (kWarps * kPairSlots) + pr) * (dv + 2);
    const int64_t stride = (int64_t)(kWarps * kPairSlots) * (dv + 2);
    // lane z (and z + 32) holds share z's maximum and denominator: all shares are read at once
    float mz[2], dz[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int z = lane + 32 * i;
      mz[i] = z < a.n_split ? w0[z * stride] : -INFINITY;
      dz[i] = z < a.n_split ? w0[z * stride + 1] : 0.f;
    }
    const float top = warp_max(fmaxf(mz[0], mz[1]));
    float fz[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) fz[i] = mz[i] == -INFINITY ? 0.f : expf(mz[i] - top);
    float den = warp_sum(dz[0] * fz[0] + dz[1] * fz[1]);
    if (a.sink) den += expf(a.sink[g * rep + pr % rep] - top);
    float o[kMaxDvLane];
#pragma unroll
    for (int e = 0; e < kMaxDvLane; ++e) o[e] = 0.f;
    for (int z0 = 0; z0 < a.n_split; z0 += 8) {   // eight shares' sums in flight
      float v[8][kMaxDvLane];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < kMaxDvLane; ++e) {
          const int c = lane + 32 * e;
          v[j][e] = (z0 + j < a.n_split && c < dv) ? w0[(z0 + j) * stride + 2 + c] : 0.f;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int z = z0 + j;   // z0 is a multiple of 8: all eight sit in the same half
        const float f = __shfl_sync(0xffffffffu, z < 32 ? fz[0] : fz[1], z & 31);
#pragma unroll
        for (int e = 0; e < kMaxDvLane; ++e) o[e] = fmaf(v[j][e], f, o[e]);
      }
    }
    const int r = pr / rep, qh = g * rep + pr % rep;
    const int64_t t = first + r;
    const float inv = a.out_scale / den;
    const float* gt = a.gate ? a.gate + t * a.ld_gate + (int64_t)qh * dv : nullptr;
    T* dst = static_cast<T*>(a.out) + t * a.ld_out + (int64_t)qh * dv;
#pragma unroll
    for (int e = 0; e < kMaxDvLane; ++e) {
      const int c = lane + 32 * e;
      if (c < dv) stf(dst + c, gt ? o[e] * inv / (1.f + expf(-gt[c])) : o[e] * inv);
    }
  }
}

inline int generic_tile_rows(int H, int G) {
  const int rep = H / G;
  if (G <= 0 || H % G || rep > kWarps * kPairSlots) return 0;
  const int t = kWarps * kPairSlots / rep;
  return t > 16 ? 16 : t;
}

inline size_t generic_smem(int d, int dv) {
  return ((size_t)kWarps * kPairSlots * d + (size_t)kKeys * (d + 1) + (size_t)kKeys * dv + kWarps * kKeys) * sizeof(float);
}

}  // namespace

extern "C" int ao_lm_qk_prep(const float* proj, int64_t ld, int64_t q_off, int64_t k_off, int64_t v_off, int64_t n, int H, int G,
                             int d, int dv, float eps, int dt, float* qn, void* kn, void* vn, void* stream) {
  LM_CHECK_ARG(proj && qn && kn && vn && n > 0 && H > 0 && G > 0 && d > 0 && dv > 0);
  LM_DISPATCH(dt, qk_prep_kernel<T><<<(unsigned)n, 128, 0, lm_stream(stream)>>>(proj, ld, q_off, k_off, v_off, H, G, d, dv, eps, qn,
                                                                                static_cast<T*>(kn), static_cast<T*>(vn)));
  return lm_launch_status();
}

extern "C" int ao_lm_qk_norm_prep(const float* proj, int64_t ld, int64_t q_off, int64_t k_off, int64_t v_off, const void* q_bias,
                                  const void* k_bias, const void* v_bias, const void* q_weight, const void* k_weight,
                                  float temp_coef, int temp_every, const int32_t* pos, const int32_t* slot, void* ring_k,
                                  void* ring_v, int ring, int64_t n, int H, int G, int d, int dv, float eps, int dt, float* qn,
                                  void* kn, void* vn, void* stream) {
  LM_CHECK_ARG(proj && qn && kn && vn && n > 0 && H > 0 && G > 0 && d > 0 && dv > 0 && (temp_coef == 0.f || (pos && temp_every > 0)));
  LM_CHECK_ARG((!ring_k && !ring_v) || (ring_k && ring_v && slot && pos && ring > 0));
  LM_DISPATCH(dt, qk_norm_prep_kernel<T><<<(unsigned)n, 128, 0, lm_stream(stream)>>>(
                      proj, ld, q_off, k_off, v_off, static_cast<const T*>(q_bias), static_cast<const T*>(k_bias),
                      static_cast<const T*>(v_bias), static_cast<const T*>(q_weight), static_cast<const T*>(k_weight), temp_coef,
                      temp_every, pos, slot, static_cast<T*>(ring_k), static_cast<T*>(ring_v), ring, H, G, d, dv, eps, qn,
                      static_cast<T*>(kn), static_cast<T*>(vn)));
  return lm_launch_status();
}

extern "C" int ao_lm_ring_append(const void* kn, const void* vn, int64_t n, int64_t k_row, int64_t v_row, int ring, int dt,
                                 const int32_t* slot, const int32_t* pos, const int32_t* ahead, void* ring_k, void* ring_v,
                                 void* stream) {
  LM_CHECK_ARG(kn && vn && slot && pos && ahead && ring_k && ring_v && n > 0 && k_row > 0 && v_row > 0 && ring > 0);
  LM_DISPATCH(dt, ring_append_kernel<T><<<(unsigned)n, 128, 0, lm_stream(stream)>>>(
                      static_cast<const T*>(kn), static_cast<const T*>(vn), k_row, v_row, ring, slot, pos, ahead,
                      static_cast<T*>(ring_k), static_cast<T*>(ring_v)));
  return lm_launch_status();
}

extern "C" int ao_lm_chunk_attention_plan(int dt, int H, int G, int d, int dv, int* tile_rows) {
  LM_CHECK_ARG(tile_rows);
  (void)dt;
  *tile_rows = (d > 0 && dv > 0 && dv <= 32 * kMaxDvLane && generic_smem(d, dv) <= 200 * 1024) ? generic_tile_rows(H, G) : 0;
  return AO_B200_OK;
}

extern "C" int64_t ao_lm_chunk_attention_workspace_bytes(int n_tiles, int G, int dv, int n_split) {
  return n_split > 1 ? (int64_t)n_tiles * G * n_split * (kWarps * kPairSlots) * (dv + 2) * 4 : 0;
}

extern "C" int ao_lm_sink_attention(const float* qn, const void* kn, const void* vn, const void* ring_k, const void* ring_v,
                                    int dt, const float* gate, int64_t ld_gate, const float* dist_bias, int n_dist,
                                    const float* sink, const int32_t* slot, const int32_t* pos, const int32_t* back,
                                    const int32_t* tile_first, const int32_t* tile_count, int n_tiles, int H, int G, int d, int dv,
                                    int chunk, float scale, float softcap, float out_scale, int n_split, void* workspace,
                                    int64_t workspace_bytes, void* out, int64_t ld_out, void* stream) {
  LM_CHECK_ARG(qn && kn && vn && ring_k && ring_v && slot && pos && back && tile_first && tile_count && out);
  LM_CHECK_ARG(n_tiles > 0 && (!dist_bias || n_dist > 0) && chunk > 0 && G > 0 && G <= 65535 && n_split >= 1 && n_split <= 64);
  if (n_split > 1) {
    LM_CHECK_ARG(workspace);
    if (workspace_bytes < ao_lm_chunk_attention_workspace_bytes(n_tiles, G, dv, n_split)) return AO_B200_ERR_WORKSPACE;
  }
  if (generic_tile_rows(H, G) == 0 || dv > 32 * kMaxDvLane) return AO_B200_ERR_UNSUPPORTED;
  const size_t smem = generic_smem(d, dv);
  if (smem > 200 * 1024) return AO_B200_ERR_UNSUPPORTED;
  ChunkArgs a{qn, kn, vn, ring_k, ring_v, gate, ld_gate, dist_bias, n_dist, sink, slot, pos, back, tile_first, tile_count,
              H, G, d, dv, chunk, scale, softcap, out_scale, out, ld_out, n_split, static_cast<float*>(workspace)};
  LM_DISPATCH(dt, {
    auto kern = chunk_attention_kernel<T>;
    if (smem > 48 * 1024) {
      static bool set = false;
      if (!set) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return AO_B200_ERR_CUDA;
        set = true;
      }
    }
    kern<<<dim3((unsigned)n_tiles, (unsigned)G, (unsigned)n_split), kWarps * 32, smem, lm_stream(stream)>>>(a);
    if (n_split > 1)
      chunk_attention_merge_kernel<T><<<dim3((unsigned)n_tiles, (unsigned)G), kWarps * 32, 0, lm_stream(stream)>>>(a);
  });
  return lm_launch_status();
}

extern "C" int ao_lm_chunk_attention(const float* qn, const void* kn, const void* vn, const void* ring_k, const void* ring_v,
                                     int dt, const float* gate, int64_t ld_gate, const float* dist_bias, int n_dist,
                                     const int32_t* slot, const int32_t* pos, const int32_t* back, const int32_t* tile_first,
                                     const int32_t* tile_count, int n_tiles, int H, int G, int d, int dv, int chunk, float scale,
                                     float softcap, float out_scale, int n_split, void* workspace, int64_t workspace_bytes,
                                     void* out, int64_t ld_out, void* stream) {
  LM_CHECK_ARG(gate && dist_bias);
  return ao_lm_sink_attention(qn, kn, vn, ring_k, ring_v, dt, gate, ld_gate, dist_bias, n_dist, nullptr, slot, pos, back,
                              tile_first, tile_count, n_tiles, H, G, d, dv, chunk, scale, softcap, out_scale, n_split, workspace,
                              workspace_bytes, out, ld_out, stream);
}
