// Softmax attention under a sliding window that also keeps the first tokens of the sequence: the query at position i sees
// key j when j <= i and (i - j < window or j < keep).  Grouped heads (H query heads over G key/value heads).  Every head may
// carry N_MAPS attention maps with queries and keys of their own over the SAME values (differential attention: two maps,
// result a_1 - lambda * a_2); the result may be divided by its root mean square over the head's values and is multiplied
// by a constant.
//
// What a sequence keeps does not grow with its length: position p lives in row p % ring of a ring (ring >= window), and
// the first `first_rows` (>= keep) positions also live in a small store of their own, where the ring's turning never
// reaches them.  A step's own keys and values are read from the step's buffers and stored AFTER every layer that reads
// the cache has run (a long prompt portion would otherwise overwrite rows that its first rows still need):
//     ao_lm_qkv_rotary_prep -> ao_lm_window_attention (this layer and the layers that borrow its keys) -> ao_lm_window_append.
// Scores, weights, the combination of the maps and the norm are fp32 in both storage types.
#include "lm_common.cuh"

using namespace lm;

namespace {

constexpr int kWarps = 8;
constexpr int kKeys = 32;        // keys per shared-memory block
constexpr int kSlots = 2;        // (row, query head) pairs per warp
constexpr int kMaxDvLane = 8;    // value size <= 32 * kMaxDvLane
constexpr int kPairs = kWarps * kSlots;

// Projection row -> biased, rotated queries (fp32 [n][q_heads][d]) and keys (storage type [n][k_heads][d]), biased values
// (storage type [n][v_width]).  k_heads == 0: a layer that borrows its keys and values projects queries only.
template <typename T>
__global__ void qkv_rotary_prep_kernel(const float* __restrict__ proj, int64_t ld, int64_t q_off, int64_t k_off, int64_t v_off,
                                       const T* __restrict__ q_bias, const T* __restrict__ k_bias, const T* __restrict__ v_bias,
                                       const int32_t* __restrict__ pos, const float* __restrict__ inv_freq, int rot_dims,
                                       int pairing, int q_heads, int k_heads, int d, int v_width, float* __restrict__ qn,
                                       T* __restrict__ kn, T* __restrict__ vn) {
  const int64_t t = blockIdx.x;
  const float p = (float)pos[t];
  const float* row = proj + t * ld;
  const int half = rot_dims / 2, per = d - half;
  const int tid = blockIdx.y * blockDim.x + threadIdx.x, nth = gridDim.y * blockDim.x;   // a row may be shared by several CTAs
  for (int i = tid; i < (q_heads + k_heads) * per; i += nth) {
    const int hd = i / per, e = i - hd * per;
    const bool is_q = hd < q_heads;
    const int64_t ho = (int64_t)(is_q ? hd : hd - q_heads) * d;
    const float* src = row + (is_q ? q_off : k_off) + ho;
    const T* bias = is_q ? q_bias : k_bias;
    float va, vb = 0.f;
    int ia, ib = -1;
    if (e < half) {
      ia = pairing ? e : 2 * e, ib = pairing ? e + half : 2 * e + 1;
      const float u = src[ia] + (bias ? ldf(bias + ho + ia) : 0.f), v = src[ib] + (bias ? ldf(bias + ho + ib) : 0.f);
      float sn, cs;
      sincosf(p * inv_freq[e], &sn, &cs);
      va = u * cs - v * sn, vb = v * cs + u * sn;
    } else {
      ia = rot_dims + (e - half);
      va = src[ia] + (bias ? ldf(bias + ho + ia) : 0.f);
    }
    if (is_q) {
      float* dst = qn + (t * q_heads + hd) * d;
      dst[ia] = va;
      if (ib >= 0) dst[ib] = vb;
    } else {
      T* dst = kn + (t * k_heads + (hd - q_heads)) * d;
      stf(dst + ia, va);
      if (ib >= 0) stf(dst + ib, vb);
    }
  }
  if (k_heads > 0)
    for (int c = tid; c < v_width; c += nth)
      stf(vn + t * v_width + c, row[v_off + c] + (v_bias ? ldf(v_bias + c) : 0.f));
}

template <typename T>
__global__ void window_append_kernel(const T* __restrict__ kn, const T* __restrict__ vn, int64_t krow, int64_t vrow, int ring,
                                     int first_rows, const int32_t* __restrict__ slot, const int32_t* __restrict__ pos,
                                     const int32_t* __restrict__ ahead, T* __restrict__ ring_k, T* __restrict__ ring_v,
                                     T* __restrict__ first_k, T* __restrict__ first_v) {
  const int64_t t = blockIdx.x;
  const int p = pos[t];
  if (ahead[t] < ring) {   // else a later row of the same step takes this ring row
    const int64_t r = (int64_t)slot[t] * ring + p % ring;
    for (int64_t c = threadIdx.x; c < krow; c += blockDim.x) ring_k[r * krow + c] = kn[t * krow + c];
    for (int64_t c = threadIdx.x; c < vrow; c += blockDim.x) ring_v[r * vrow + c] = vn[t * vrow + c];
  }
  if (p < first_rows) {
    const int64_t r = (int64_t)slot[t] * first_rows + p;
    for (int64_t c = threadIdx.x; c < krow; c += blockDim.x) first_k[r * krow + c] = kn[t * krow + c];
    for (int64_t c = threadIdx.x; c < vrow; c += blockDim.x) first_v[r * vrow + c] = vn[t * vrow + c];
  }
}

struct WinArgs {
  const float* qn;                 // [n][H][NM][d]
  const void *kn, *vn;             // the step's rows [n][G][NM][d], [n][G][dv]
  const void *ring_k, *ring_v;     // [slots][ring][G][NM d], [slots][ring][G][dv]
  const void *first_k, *first_v;   // [slots][first_rows][...]
  int ring, first_rows;
  const int32_t *slot, *pos, *back, *tile_first, *tile_count;
  int H, G, d, dv, window, keep;
  float scale, lambda, out_scale, eps;
  int unit_rms;
  void* out;                       // [n][ld_out], H * dv per row
  int64_t ld_out;
  int n_split;                     // > 1: blockIdx.z takes a share of the key blocks and leaves (max, denominator, sums) in ws
  int vec16;                       // rows of keys and values are whole 16-byte pieces on 16-byte boundaries: staged 16 bytes at a time
  float* ws;                       // [tiles][G * head shares][n_split][kPairs][n_maps][dv + 2]
};

// a_1 - lambda a_2 (or a_1 alone), optionally divided by its root mean square over the head's dv values, times out_scale:
// what a warp does with the normalised sums of its (row, query head) pair, lane = value column mod 32.
template <typename T, int NM>
__device__ __forceinline__ void finish_pair(const WinArgs& a, const float (&av)[NM][kMaxDvLane], int lane, T* dst) {
  float val[kMaxDvLane], ss = 0.f;
#pragma unroll
  for (int e = 0; e < kMaxDvLane; ++e) {
    float v = av[0][e];
    if (NM == 2) v -= a.lambda * av[NM - 1][e];
    val[e] = lane + 32 * e < a.dv ? v : 0.f;
    ss = fmaf(val[e], val[e], ss);
  }
  float k = a.out_scale;
  if (a.unit_rms) k /= sqrtf(warp_sum(ss) / (float)a.dv + a.eps);
#pragma unroll
  for (int e = 0; e < kMaxDvLane; ++e) {
    const int c = lane + 32 * e;
    if (c < a.dv) stf(dst + c, val[e] * k);
  }
}

// kKeys rows of `width` values (storage type, 16-byte aligned rows, width a multiple of a 16-byte piece) -> fp32 in shared
// memory, row jj at dst + jj * stride; rows at or past nk become zeros.  A thread's pieces (up to four) are all in flight
// before the first is stored: a decoded token's CTA otherwise waits for one DRAM round trip per element it fetches.
template <typename T, typename RowOf>
__device__ __forceinline__ void stage_key_block(float* dst, int stride, int width, int k0, int nk, RowOf row_of) {
  constexpr int kPer = 16 / (int)sizeof(T), kFlight = 4;
  const int per_row = width / kPer, total = kKeys * per_row;
  for (int base = 0; base < total; base += kFlight * blockDim.x) {
    uint4 v[kFlight];
#pragma unroll
    for (int u = 0; u < kFlight; ++u) {
      const int i = base + u * blockDim.x + threadIdx.x;
      v[u] = make_uint4(0, 0, 0, 0);
      if (i < total) {
        const int jj = i / per_row, kk = k0 + jj;
        if (kk < nk) v[u] = __ldg(reinterpret_cast<const uint4*>(row_of(kk)) + (i - jj * per_row));
      }
    }
#pragma unroll
    for (int u = 0; u < kFlight; ++u) {
      const int i = base + u * blockDim.x + threadIdx.x;
      if (i < total) {
        const int jj = i / per_row;
        unpack16(v[u], dst + (size_t)jj * stride + (size_t)(i - jj * per_row) * kPer, static_cast<const T*>(nullptr));
      }
    }
  }
}

// One CTA = a tile of consecutive rows of one segment x one key/value head (a group of more than kPairs query heads is
// shared out over several CTAs of one row each); a warp owns up to kSlots (row, query head) pairs and keeps the running
// maximum, denominator and sums of all their maps in registers.  Key index kk of the tile
// enumerates the kept first positions that lie in front of the tile's window, then the window from its first row's
// oldest key to its last row's own position.
template <typename T, int NM>
__global__ void __launch_bounds__(kWarps * 32) window_attention_kernel(WinArgs a) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x;
  const int d = a.d, dv = a.dv, G = a.G;
  const int rep_all = a.H / G, rep = min(rep_all, kPairs), subs = (rep_all + rep - 1) / rep;
  const int g = blockIdx.y / subs, h_first = (blockIdx.y % subs) * rep;    // this CTA's query heads of the group: h_first .. + rep
  const int first = a.tile_first[tile], count = a.tile_count[tile];
  const int pa = a.pos[first], back0 = a.back[first];
  const int p0 = pa - back0;                          // the first position the step brings of this sequence
  const int64_t seg_row0 = first - back0;
  const int lo = max(0, pa - a.window + 1);
  const int nf = min(a.keep, lo);
  const int nk = nf + (pa + count - lo);
  const int npairs = count * rep;
  const int KD = NM * d, KP = KD + 1;
  float* Qs = sm;                                     // [kPairs][NM d]
  float* Ks = Qs + (size_t)kPairs * KD;               // [kKeys][NM d + 1]
  float* Vs = Ks + (size_t)kKeys * KP;                // [kKeys][dv]
  float* Ps = Vs + (size_t)kKeys * dv;                // [kWarps][NM][kKeys]
  const int64_t s = a.slot[first];
  const T* ring_k = static_cast<const T*>(a.ring_k) + (s * a.ring * G + g) * KD;
  const T* ring_v = static_cast<const T*>(a.ring_v) + (s * a.ring * G + g) * dv;
  const T* first_k = static_cast<const T*>(a.first_k) + (s * a.first_rows * G + g) * KD;
  const T* first_v = static_cast<const T*>(a.first_v) + (s * a.first_rows * G + g) * dv;
  const T* step_k = static_cast<const T*>(a.kn) + (seg_row0 * G + g) * KD;
  const T* step_v = static_cast<const T*>(a.vn) + (seg_row0 * G + g) * dv;

  for (int i = threadIdx.x; i < npairs * KD; i += blockDim.x) {
    const int pr = i / KD, c = i - pr * KD, r = pr / rep, hq = h_first + pr % rep;
    Qs[i] = hq < rep_all ? a.qn[((int64_t)(first + r) * a.H + g * rep_all + hq) * KD + c] : 0.f;
  }
  float mx[kSlots][NM], den[kSlots][NM], o[kSlots][NM][kMaxDvLane];
#pragma unroll
  for (int sl = 0; sl < kSlots; ++sl)
#pragma unroll
    for (int m = 0; m < NM; ++m) {
      mx[sl][m] = -INFINITY, den[sl][m] = 0.f;
#pragma unroll
      for (int e = 0; e < kMaxDvLane; ++e) o[sl][m][e] = 0.f;
    }
  const int blocks = (nk + kKeys - 1) / kKeys, per = (blocks + a.n_split - 1) / a.n_split;
  const int k_begin = blockIdx.z * per * kKeys, k_end = min(nk, (int)(blockIdx.z + 1) * per * kKeys);
  for (int k0 = k_begin; k0 < k_end; k0 += kKeys) {
    __syncthreads();   // the previous block is used up (and, the first time, the queries are in place)
    if (a.vec16) {
      stage_key_block<T>(Ks, KP, KD, k0, nk, [&](int kk) {
        const int j = kk < nf ? kk : lo + (kk - nf);
        return j >= p0 ? step_k + (int64_t)(j - p0) * G * KD
                       : (j < a.first_rows ? first_k + (int64_t)j * G * KD : ring_k + (int64_t)(j % a.ring) * G * KD);
      });
      stage_key_block<T>(Vs, dv, dv, k0, nk, [&](int kk) {
        const int j = kk < nf ? kk : lo + (kk - nf);
        return j >= p0 ? step_v + (int64_t)(j - p0) * G * dv
                       : (j < a.first_rows ? first_v + (int64_t)j * G * dv : ring_v + (int64_t)(j % a.ring) * G * dv);
      });
    } else {
      for (int i = threadIdx.x; i < kKeys * KD; i += blockDim.x) {
        const int jj = i / KD, c = i - jj * KD, kk = k0 + jj;
        float v = 0.f;
        if (kk < nk) {
          const int j = kk < nf ? kk : lo + (kk - nf);
          const T* src = j >= p0 ? step_k + (int64_t)(j - p0) * G * KD
                                 : (j < a.first_rows ? first_k + (int64_t)j * G * KD : ring_k + (int64_t)(j % a.ring) * G * KD);
          v = ldf(src + c);
        }
        Ks[jj * KP + c] = v;
      }
      for (int i = threadIdx.x; i < kKeys * dv; i += blockDim.x) {
        const int jj = i / dv, c = i - jj * dv, kk = k0 + jj;
        float v = 0.f;
        if (kk < nk) {
          const int j = kk < nf ? kk : lo + (kk - nf);
          const T* src = j >= p0 ? step_v + (int64_t)(j - p0) * G * dv
                                 : (j < a.first_rows ? first_v + (int64_t)j * G * dv : ring_v + (int64_t)(j % a.ring) * G * dv);
          v = ldf(src + c);
        }
        Vs[jj * dv + c] = v;
      }
    }
    __syncthreads();
    const int kk = k0 + lane;
    const int j = kk < nf ? kk : lo + (kk - nf);                    // this lane's key position
    const int j_lo = k0 < nf ? k0 : lo + (k0 - nf);                 // the block's first and last positions
    const int kl = min(k0 + kKeys, nk) - 1;
    const int j_hi = kl < nf ? kl : lo + (kl - nf);
#pragma unroll
    for (int sl = 0; sl < kSlots; ++sl) {
      const int pr = warp + sl * kWarps;
      if (pr >= npairs || h_first + pr % rep >= rep_all) continue;    // uniform over the warp
      const int i_pos = pa + pr / rep;
      if (j_lo > i_pos) continue;                      // the whole block lies in the row's future
      if (k0 >= nf && j_hi <= i_pos - a.window && j_lo >= a.keep) continue;   // ... or behind its window
      const bool seen = kk < nk && j <= i_pos && (i_pos - j < a.window || j < a.keep);
      const float* q = Qs + (size_t)pr * KD;
      const float* kr = Ks + (size_t)lane * KP;
      float sc[NM], corr[NM];
      bool any = false;
#pragma unroll
      for (int m = 0; m < NM; ++m) {
        float acc = 0.f;
        for (int c = 0; c < d; ++c) acc = fmaf(q[m * d + c], kr[m * d + c], acc);
        sc[m] = seen ? acc * a.scale : -INFINITY;
        const float top = fmaxf(mx[sl][m], warp_max(sc[m]));
        if (top == -INFINITY) {                        // no key of the block is seen by this row (uniform)
          corr[m] = 1.f;
          Ps[(warp * NM + m) * kKeys + lane] = 0.f;
          continue;
        }
        any = true;
        corr[m] = mx[sl][m] == -INFINITY ? 0.f : expf(mx[sl][m] - top);
        const float p = expf(sc[m] - top);
        mx[sl][m] = top;
        den[sl][m] = den[sl][m] * corr[m] + warp_sum(p);
        Ps[(warp * NM + m) * kKeys + lane] = p;
      }
      __syncwarp();
      if (any) {
#pragma unroll
        for (int e = 0; e < kMaxDvLane; ++e) {
          const int c = lane + 32 * e;
          if (c < dv) {
            float acc[NM];
#pragma unroll
            for (int m = 0; m < NM; ++m) acc[m] = o[sl][m][e] * corr[m];
            for (int jj = 0; jj < kKeys; ++jj) {
              const float v = Vs[jj * dv + c];
#pragma unroll
              for (int m = 0; m < NM; ++m) acc[m] = fmaf(Ps[(warp * NM + m) * kKeys + jj], v, acc[m]);
            }
#pragma unroll
            for (int m = 0; m < NM; ++m) o[sl][m][e] = acc[m];
          }
        }
      }
      __syncwarp();
    }
  }
#pragma unroll
  for (int sl = 0; sl < kSlots; ++sl) {
    const int pr = warp + sl * kWarps;
    if (pr >= npairs || h_first + pr % rep >= rep_all) continue;
    if (a.n_split > 1) {   // this share's maximum, denominator and sums; the merge kernel finishes the pair
#pragma unroll
      for (int m = 0; m < NM; ++m) {
        float* w = a.ws + (((((int64_t)tile * gridDim.y + blockIdx.y) * a.n_split + blockIdx.z) * kPairs + pr) * NM + m) * (dv + 2);
        if (lane == 0) w[0] = mx[sl][m], w[1] = den[sl][m];
#pragma unroll
        for (int e = 0; e < kMaxDvLane; ++e)
          if (lane + 32 * e < dv) w[2 + lane + 32 * e] = o[sl][m][e];
      }
      continue;
    }
    const int r = pr / rep, qh = g * rep_all + h_first + pr % rep;
    float av[NM][kMaxDvLane];
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
      for (int e = 0; e < kMaxDvLane; ++e) av[m][e] = o[sl][m][e] / den[sl][m];
    finish_pair<T, NM>(a, av, lane, static_cast<T*>(a.out) + (int64_t)(first + r) * a.ld_out + (int64_t)qh * dv);
  }
}

// The shares of the key splits, merged on a common maximum per (pair, map), then finished like an unsplit pair.
// One CTA per (tile, key/value head, pair): warp w merges shares w, w + 8, ... (all their loads in flight at once) and
// leaves its (maximum, denominator, sums) in shared memory; a thread per value column merges the eight; warp 0 finishes.
template <typename T, int NM>
__global__ void __launch_bounds__(kWarps * 32) window_attention_merge_kernel(WinArgs a) {
  extern __shared__ float sm[];    // [kWarps][NM][dv + 2], then [NM][dv]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, pr = blockIdx.z;
  const int dv = a.dv;
  const int rep_all = a.H / a.G, rep = min(rep_all, kPairs), subs = (rep_all + rep - 1) / rep;
  const int g = blockIdx.y / subs, h_first = (blockIdx.y % subs) * rep;
  const int first = a.tile_first[tile], npairs = a.tile_count[tile] * rep;
  if (pr >= npairs || h_first + pr % rep >= rep_all) return;
  const int64_t stride = (int64_t)kPairs * NM * (dv + 2);          // from one share to the next
  constexpr int kPer = 64 / kWarps;                                // shares per warp at most
  float* part = sm;
  float* fin = sm + (size_t)kWarps * NM * (dv + 2);
#pragma unroll
  for (int m = 0; m < NM; ++m) {
    const float* w0 = a.ws + (((((int64_t)tile * gridDim.y + blockIdx.y) * a.n_split) * kPairs + pr) * NM + m) * (dv + 2);
    float mz[kPer], dz[kPer], v[kPer][kMaxDvLane];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int z = warp + j * kWarps;
      const bool in = z < a.n_split;
      mz[j] = in ? w0[z * stride] : -INFINITY;
      dz[j] = in ? w0[z * stride + 1] : 0.f;
#pragma unroll
      for (int e = 0; e < kMaxDvLane; ++e) v[j][e] = (in && lane + 32 * e < dv) ? w0[z * stride + 2 + lane + 32 * e] : 0.f;
    }
    float top = -INFINITY;
#pragma unroll
    for (int j = 0; j < kPer; ++j) top = fmaxf(top, mz[j]);
    float den = 0.f, acc[kMaxDvLane];
#pragma unroll
    for (int e = 0; e < kMaxDvLane; ++e) acc[e] = 0.f;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const float f = mz[j] == -INFINITY ? 0.f : expf(mz[j] - top);     // a share that saw no key weighs nothing
      den = fmaf(dz[j], f, den);
#pragma unroll
      for (int e = 0; e < kMaxDvLane; ++e) acc[e] = fmaf(v[j][e], f, acc[e]);
    }
    float* mine = part + ((size_t)warp * NM + m) * (dv + 2);
    if (lane == 0) mine[0] = top, mine[1] = den;
#pragma unroll
    for (int e = 0; e < kMaxDvLane; ++e)
      if (lane + 32 * e < dv) mine[2 + lane + 32 * e] = acc[e];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < NM * dv; i += blockDim.x) {
    const int m = i / dv, c = i - m * dv;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) top = fmaxf(top, part[((size_t)w * NM + m) * (dv + 2)]);
    float den = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float* pw = part + ((size_t)w * NM + m) * (dv + 2);
      const float f = pw[0] == -INFINITY ? 0.f : expf(pw[0] - top);
      den = fmaf(pw[1], f, den);
      acc = fmaf(pw[2 + c], f, acc);
    }
    fin[i] = acc / den;
  }
  __syncthreads();
  if (warp == 0) {
    float av[NM][kMaxDvLane];
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
      for (int e = 0; e < kMaxDvLane; ++e) av[m][e] = lane + 32 * e < dv ? fin[m * dv + lane + 32 * e] : 0.f;
    const int r = pr / rep, qh = g * rep_all + h_first + pr % rep;
    finish_pair<T, NM>(a, av, lane, static_cast<T*>(a.out) + (int64_t)(first + r) * a.ld_out + (int64_t)qh * dv);
  }
}

inline int win_tile_rows(int H, int G) {
  if (G <= 0 || H % G) return 0;
  return H / G > kPairs ? 1 : kPairs / (H / G);
}
// CTAs that share out the query heads of one key/value head
inline int win_head_shares(int H, int G) { return H / G > kPairs ? (H / G + kPairs - 1) / kPairs : 1; }
inline size_t win_smem(int nm, int d, int dv) {
  return ((size_t)kPairs * nm * d + (size_t)kKeys * (nm * d + 1) + (size_t)kKeys * dv + (size_t)kWarps * nm * kKeys) * sizeof(float);
}

template <typename T, int NM>
int launch_window(const WinArgs& a, int n_tiles, size_t smem, cudaStream_t st) {
  auto kern = window_attention_kernel<T, NM>;
  if (smem > 48 * 1024) {
    static bool set = false;   // per instantiation
    if (!set) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return AO_B200_ERR_CUDA;
      set = true;
    }
  }
  const unsigned gy = (unsigned)(a.G * win_head_shares(a.H, a.G));
  kern<<<dim3((unsigned)n_tiles, gy, (unsigned)a.n_split), kWarps * 32, smem, st>>>(a);
  if (a.n_split > 1) {
    const size_t msm = ((size_t)kWarps * NM * (a.dv + 2) + (size_t)NM * a.dv) * sizeof(float);      // <= 19 KB
    window_attention_merge_kernel<T, NM><<<dim3((unsigned)n_tiles, gy, kPairs), kWarps * 32, msm, st>>>(a);
  }
  return lm_launch_status();
}

}  // namespace

extern "C" int ao_lm_qkv_rotary_prep(const float* proj, int64_t ld, int64_t q_off, int64_t k_off, int64_t v_off, const void* q_bias,
                                     const void* k_bias, const void* v_bias, const int32_t* pos, const float* inv_freq,
                                     int rot_dims, int pairing, int64_t n, int q_heads, int k_heads, int d, int v_width, int dt,
                                     float* qn, void* kn, void* vn, void* stream) {
  LM_CHECK_ARG(proj && pos && qn && n > 0 && q_heads > 0 && k_heads >= 0 && d > 0 && (k_heads == 0 || (kn && vn && v_width > 0)));
  LM_CHECK_ARG(rot_dims >= 0 && rot_dims <= d && rot_dims % 2 == 0 && (rot_dims == 0 || inv_freq) && (pairing == 0 || pairing == 1));
  // few rows (decoded tokens): several CTAs per row, so that no thread walks more than a few coordinates
  const int64_t items = (int64_t)(q_heads + k_heads) * (d - rot_dims / 2);
  const int64_t room = (592 + n - 1) / n, want = (items + 511) / 512;
  const unsigned parts = n < 296 ? (unsigned)(want > room ? room : want < 1 ? 1 : want) : 1u;
  LM_DISPATCH(dt, qkv_rotary_prep_kernel<T><<<dim3((unsigned)n, parts), 256, 0, lm_stream(stream)>>>(
                      proj, ld, q_off, k_off, v_off, static_cast<const T*>(q_bias), static_cast<const T*>(k_bias),
                      static_cast<const T*>(v_bias), pos, inv_freq, rot_dims, pairing, q_heads, k_heads, d, v_width, qn,
                      static_cast<T*>(kn), static_cast<T*>(vn)));
  return lm_launch_status();
}

extern "C" int ao_lm_window_append(const void* kn, const void* vn, int64_t n, int64_t k_row, int64_t v_row, int ring,
                                   int first_rows, int dt, const int32_t* slot, const int32_t* pos, const int32_t* ahead,
                                   void* ring_k, void* ring_v, void* first_k, void* first_v, void* stream) {
  LM_CHECK_ARG(kn && vn && slot && pos && ahead && ring_k && ring_v && n > 0 && k_row > 0 && v_row > 0 && ring > 0 && first_rows >= 0);
  LM_CHECK_ARG(first_rows == 0 || (first_k && first_v));
  LM_DISPATCH(dt, window_append_kernel<T><<<(unsigned)n, 128, 0, lm_stream(stream)>>>(
                      static_cast<const T*>(kn), static_cast<const T*>(vn), k_row, v_row, ring, first_rows, slot, pos, ahead,
                      static_cast<T*>(ring_k), static_cast<T*>(ring_v), static_cast<T*>(first_k), static_cast<T*>(first_v)));
  return lm_launch_status();
}

extern "C" int64_t ao_lm_window_attention_workspace_bytes(int n_tiles, int n_maps, int H, int G, int dv, int n_split) {
  if (n_split <= 1 || G <= 0 || H % G) return 0;
  return (int64_t)n_tiles * G * win_head_shares(H, G) * n_split * kPairs * n_maps * (dv + 2) * 4;
}

extern "C" int ao_lm_window_attention_plan(int dt, int n_maps, int H, int G, int d, int dv, int* tile_rows) {
  LM_CHECK_ARG(tile_rows);
  (void)dt;
  const bool ok = (n_maps == 1 || n_maps == 2) && d > 0 && dv > 0 && dv <= 32 * kMaxDvLane && win_smem(n_maps, d, dv) <= 200 * 1024;
  *tile_rows = ok ? win_tile_rows(H, G) : 0;
  return AO_B200_OK;
}

extern "C" int ao_lm_window_attention(const float* qn, const void* kn, const void* vn, const void* ring_k, const void* ring_v,
                                      const void* first_k, const void* first_v, int ring, int first_rows, int dt,
                                      const int32_t* slot, const int32_t* pos, const int32_t* back, const int32_t* tile_first,
                                      const int32_t* tile_count, int n_tiles, int n_maps, int H, int G, int d, int dv, int window,
                                      int keep, float scale, float lambda, int unit_rms, float eps, float out_scale, int n_split,
                                      void* workspace, int64_t workspace_bytes, void* out, int64_t ld_out, void* stream) {
  LM_CHECK_ARG(qn && kn && vn && ring_k && ring_v && slot && pos && back && tile_first && tile_count && out);
  LM_CHECK_ARG(n_tiles > 0 && window > 0 && keep >= 0 && ring >= window && first_rows >= keep && (first_rows == 0 || (first_k && first_v)));
  LM_CHECK_ARG(G > 0 && H > 0 && H <= 65535 && (n_maps == 1 || n_maps == 2) && n_split >= 1 && n_split <= 64);
  if (n_split > 1) {
    LM_CHECK_ARG(workspace);
    if (workspace_bytes < ao_lm_window_attention_workspace_bytes(n_tiles, n_maps, H, G, dv, n_split)) return AO_B200_ERR_WORKSPACE;
  }
  if (win_tile_rows(H, G) == 0 || dv > 32 * kMaxDvLane) return AO_B200_ERR_UNSUPPORTED;
  const size_t smem = win_smem(n_maps, d, dv);
  if (smem > 200 * 1024) return AO_B200_ERR_UNSUPPORTED;
  const int piece = dt == AO_LM_BF16 ? 8 : 4;    // values of the storage type in 16 bytes
  auto on16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const int vec16 = (n_maps * d) % piece == 0 && dv % piece == 0 && on16(kn) && on16(vn) && on16(ring_k) && on16(ring_v) &&
                    (!first_k || on16(first_k)) && (!first_v || on16(first_v));
  WinArgs a{qn, kn, vn, ring_k, ring_v, first_k ? first_k : ring_k, first_v ? first_v : ring_v, ring, first_rows, slot, pos, back,
            tile_first, tile_count, H, G, d, dv, window, keep, scale, lambda, out_scale, eps, unit_rms, out, ld_out, n_split, vec16,
            static_cast<float*>(workspace)};
  const cudaStream_t st = lm_stream(stream);
  LM_DISPATCH(dt, {
    if (n_maps == 2) return launch_window<T, 2>(a, n_tiles, smem, st);
    return launch_window<T, 1>(a, n_tiles, smem, st);
  });
  return AO_B200_OK;
}
