// Recurrences whose state is a matrix per head, S_t = a_t S_(t-1) + b_t k_t v_t^T (S: d x dv), read out as
// o_t = S_t^T q_t + skip_h v_t.  Two mixers are this recurrence with different decays:
//   linear attention with a fixed decay per head     a_t = decay_h, b_t = 1, q / k / v through an activation;
//   state-space duality (selective state space)      a_t = exp(-exp(A_h) dt_t), b_t = dt_t, k = B_t, q = C_t shared by the
//                                                    heads of a group, v = x_t, skip_h = D_h,
// so one kernel serves both, with a and b per (row, head) in device memory or constant per head.
//
// The state lives in fp32 [slots][H][d][dv] and is carried from step to step; a sequence that starts at position 0 starts
// from zeros without reading its slot.  Every product and sum is fp32, and every token is folded into the state by the
// same instructions whether it arrives alone or inside a prompt portion, so a result does not depend on how the sequence
// was cut into steps.
//
// One CTA = one segment (consecutive rows of one sequence) x one head x 32 or 64 value columns.  Lane = one or two
// columns, warp p owns DR rows of the state in registers; tokens are staged 16 at a time in shared memory, each warp leaves its partial read-outs
// there and the block adds them up once per 16 tokens.  A segment longer than a tile runs in three launches instead: every
// tile from a zero state, the tiles' start states carried through the segment element by element, and the read-out of
// each tile's start state added to its rows (same sums, another order).
//
// Around it: the input side of the state-space mixer (causal convolution over time with the slot's memory + SiLU,
// softplus step sizes, decays), the convolution memory's update, and the gated group RMS norm both mixers end with.
#include "lm_common.cuh"

using namespace lm;

namespace {

constexpr int kTB = 16;        // tokens staged per round

__device__ __forceinline__ float act_apply(float v, int act) { return act == 1 ? v / (1.f + expf(-v)) : v; }

struct RecArgs {
  const float *q, *k, *v;        // rows [n][ld*]; q / k hold G groups of d, v holds H heads of dv
  int64_t ldq, ldk, ldv;
  int act;                       // 0: as they are, 1: SiLU on load
  const float *a, *b;            // [n][ld_ab] per (row, head); null: a = a_head[h], b = 1
  int64_t ld_ab;
  const float *a_head, *skip;    // [H]; skip null: none
  int H, G, d, dv;
  float* state;                  // [slots][H][d][dv]
  const int32_t *slot, *pos, *seg_first, *seg_count;   // whole segments, or (tiled form) tiles of rows inside segments
  float* out;                    // [n][ld_out], H * dv per row
  int64_t ld_out;
  // tiled form: per tile the state it builds from zero, the state it starts from, and per row the product of the decays
  // from its tile's first row on
  float *ws_local, *ws_start, *pcum;
  const int32_t *seg_tile0, *seg_tiles;
};

// rows [row0, row0 + nb) of src (row stride ld, `wd` values per row) -> dst[j][wp], zeros beyond wd; a warp per row
__device__ __forceinline__ void stage_rows(const float* __restrict__ src, int64_t ld, int64_t row0, int nb, int wd, int wp,
                                           int act, float* __restrict__ dst) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const bool vec = (wd & 3) == 0 && (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  for (int j = warp; j < nb; j += nw) {
    const float* r = src + (row0 + j) * ld;
    float* o = dst + j * wp;
    if (vec) {
      for (int e = lane * 4; e < wp; e += 128) {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (e < wd) {
          x = *reinterpret_cast<const float4*>(r + e);
          x.x = act_apply(x.x, act), x.y = act_apply(x.y, act), x.z = act_apply(x.z, act), x.w = act_apply(x.w, act);
        }
        *reinterpret_cast<float4*>(o + e) = x;
      }
    } else {
      for (int e = lane; e < wp; e += 32) o[e] = e < wd ? act_apply(r[e], act) : 0.f;
    }
  }
}

// MODE 0: whole segments on the slots' state.  MODE 1 (tiled form, first pass): a tile of rows from a zero state; the
// state it ends with goes to ws_local, the running product of its decays to pcum.  MODE 2 (third pass): the read-out of
// the state the tile starts from (ws_start, made by the carry pass), scaled by the decays up to each row, added to out.
template <int DR, int MODE, int NC>   // NC value columns per lane: a CTA covers 32 NC columns
__global__ void __launch_bounds__(DR == 32 ? 1024 : 256, DR == 32 ? 1 : (NC == 2 ? 2 : 4)) outer_recurrence_kernel(RecArgs A) {
  constexpr int KC = 32 * NC;
  extern __shared__ __align__(16) float sm[];
  const int P = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dp = P * DR;                       // d rounded up to what the warps cover
  float* qs = sm;                              // [kTB][dp]
  float* ks = qs + kTB * dp;                   // [kTB][dp]
  float* vs = ks + kTB * dp;                   // [kTB][KC]
  float* ab = vs + kTB * KC;                // [kTB][2]
  float* op = ab + kTB * 2;                    // [P][kTB][KC]
  const int seg = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * KC;
  const int first = A.seg_first[seg], count = A.seg_count[seg];
  const int g = h / (A.H / A.G), d = A.d, dv = A.dv;
  float* srow = MODE == 0 ? A.state + (((int64_t)A.slot[first] * A.H + h) * d) * dv
                          : (MODE == 1 ? A.ws_local : A.ws_start) + (((int64_t)seg * A.H + h) * d) * dv;
  float S[NC][DR];
  const bool fresh = MODE == 1 || (MODE == 0 && A.pos[first] == 0);
#pragma unroll
  for (int cc = 0; cc < NC; ++cc) {
    const int c = c0 + 32 * cc + lane;
#pragma unroll
    for (int r = 0; r < DR; ++r) {
      const int i = warp * DR + r;
      S[cc][r] = (!fresh && c < dv && i < d) ? srow[(int64_t)i * dv + c] : 0.f;
    }
  }
  const float skip = (MODE != 2 && A.skip) ? A.skip[h] : 0.f;
  if (MODE == 1 && blockIdx.z == 0 && threadIdx.x == 0) {   // the decays' running product, once per (tile, head)
    float pr = 1.f;
    for (int j = 0; j < count; ++j) {
      pr *= A.a ? A.a[(int64_t)(first + j) * A.ld_ab + h] : A.a_head[h];
      A.pcum[(int64_t)(first + j) * A.H + h] = pr;
    }
  }
  const float* qg = A.q + (int64_t)g * d;
  const float* kg = A.k + (int64_t)g * d;
  // Common shapes (8 warps, 16-byte rows): the next round's rows travel from global memory into registers while this
  // round is computed, so no warp waits for them at the top of a round (in the read-out pass: the rows' old results and decay
  // products as well).
  const bool piped = DR <= 16 && P == 8 && count > kTB && (d & 3) == 0 && (A.ldq & 3) == 0 && (reinterpret_cast<uintptr_t>(qg) & 15) == 0 &&
                     (MODE == 2 || ((A.ldk & 3) == 0 && (reinterpret_cast<uintptr_t>(kg) & 15) == 0));
  // one round = up to kTB staged tokens: every warp folds them into its rows of the state and leaves partial read-outs
  auto compute_round = [&](int nb) {
    for (int j = 0; j < nb; ++j) {
      const float4* q4 = reinterpret_cast<const float4*>(qs + j * dp + warp * DR);
      float o[NC][4];   // four chains per column: the read-out does not wait on one accumulator
#pragma unroll
      for (int cc = 0; cc < NC; ++cc) o[cc][0] = o[cc][1] = o[cc][2] = o[cc][3] = 0.f;
      if (MODE != 2) {
        const float a = ab[2 * j];
        float bv[NC];
#pragma unroll
        for (int cc = 0; cc < NC; ++cc) bv[cc] = ab[2 * j + 1] * vs[j * KC + 32 * cc + lane];
        const float4* k4 = reinterpret_cast<const float4*>(ks + j * dp + warp * DR);
#pragma unroll
        for (int r4 = 0; r4 < DR / 4; ++r4) {
          const float4 kk = k4[r4], qq = q4[r4];   // one pair of loads serves every column of the lane
#pragma unroll
          for (int cc = 0; cc < NC; ++cc) {
            S[cc][4 * r4 + 0] = fmaf(a, S[cc][4 * r4 + 0], kk.x * bv[cc]);
            S[cc][4 * r4 + 1] = fmaf(a, S[cc][4 * r4 + 1], kk.y * bv[cc]);
            S[cc][4 * r4 + 2] = fmaf(a, S[cc][4 * r4 + 2], kk.z * bv[cc]);
            S[cc][4 * r4 + 3] = fmaf(a, S[cc][4 * r4 + 3], kk.w * bv[cc]);
            o[cc][0] = fmaf(S[cc][4 * r4 + 0], qq.x, o[cc][0]);
            o[cc][1] = fmaf(S[cc][4 * r4 + 1], qq.y, o[cc][1]);
            o[cc][2] = fmaf(S[cc][4 * r4 + 2], qq.z, o[cc][2]);
            o[cc][3] = fmaf(S[cc][4 * r4 + 3], qq.w, o[cc][3]);
          }
        }
      } else {
#pragma unroll
        for (int r4 = 0; r4 < DR / 4; ++r4) {
          const float4 qq = q4[r4];
#pragma unroll
          for (int cc = 0; cc < NC; ++cc) {
            o[cc][0] = fmaf(S[cc][4 * r4 + 0], qq.x, o[cc][0]);
            o[cc][1] = fmaf(S[cc][4 * r4 + 1], qq.y, o[cc][1]);
            o[cc][2] = fmaf(S[cc][4 * r4 + 2], qq.z, o[cc][2]);
            o[cc][3] = fmaf(S[cc][4 * r4 + 3], qq.w, o[cc][3]);
          }
        }
      }
#pragma unroll
      for (int cc = 0; cc < NC; ++cc)
        op[(warp * kTB + j) * KC + 32 * cc + lane] = (o[cc][0] + o[cc][1]) + (o[cc][2] + o[cc][3]);
    }
  };
  auto reduce_round = [&](int t0, int nb) {
    for (int i = threadIdx.x; i < nb * KC; i += blockDim.x) {
      const int j = i / KC, e = i - j * KC;
      if (c0 + e >= dv) continue;
      float o = 0.f;
      for (int p = 0; p < P; ++p) o += op[(p * kTB + j) * KC + e];
      float* dst = A.out + (int64_t)(first + t0 + j) * A.ld_out + (int64_t)h * dv + c0 + e;
      if (MODE == 2)
        *dst = piped ? fmaf(ab[2 * j], o, vs[i]) : *dst + A.pcum[(int64_t)(first + t0 + j) * A.H + h] * o;
      else
        *dst = fmaf(skip, vs[i], o);
    }
  };
  if (piped) {
    float4 rq[2], rk[2];
    float rv[2 * NC], ra = 0.f, rb = 1.f;
    const int e4 = lane * 4;
    auto fetch = [&](int t0, int nb) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int j = warp + 8 * r;
        rq[r] = rk[r] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < nb && e4 < d) {
          rq[r] = *reinterpret_cast<const float4*>(qg + (int64_t)(first + t0 + j) * A.ldq + e4);
          if (MODE != 2) rk[r] = *reinterpret_cast<const float4*>(kg + (int64_t)(first + t0 + j) * A.ldk + e4);
        }
      }
#pragma unroll
      for (int r = 0; r < 2 * NC; ++r) {     // values, or (read-out pass) what the rows hold so far
        const int i = threadIdx.x + 256 * r, jv = i / KC, ev = i - jv * KC;
        const float* src = MODE != 2 ? A.v + (int64_t)(first + t0 + jv) * A.ldv : A.out + (int64_t)(first + t0 + jv) * A.ld_out;
        rv[r] = (jv < nb && c0 + ev < dv) ? src[(int64_t)h * dv + c0 + ev] : 0.f;
      }
      if ((int)threadIdx.x < nb) {
        const int64_t t = first + t0 + threadIdx.x;
        if (MODE != 2) {
          ra = A.a ? A.a[t * A.ld_ab + h] : A.a_head[h];
          rb = A.b ? A.b[t * A.ld_ab + h] : 1.f;
        } else {
          ra = A.pcum[t * A.H + h];
        }
      }
    };
    auto act4 = [&](float4 x) {
      x.x = act_apply(x.x, A.act), x.y = act_apply(x.y, A.act), x.z = act_apply(x.z, A.act), x.w = act_apply(x.w, A.act);
      return x;
    };
    fetch(0, min(kTB, count));
    for (int t0 = 0; t0 < count; t0 += kTB) {
      const int nb = min(kTB, count - t0);
      __syncthreads();   // the previous round's read-outs are out
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int j = warp + 8 * r;
        if (e4 < dp) {
          *reinterpret_cast<float4*>(qs + j * dp + e4) = act4(rq[r]);
          if (MODE != 2) *reinterpret_cast<float4*>(ks + j * dp + e4) = act4(rk[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < 2 * NC; ++r) vs[threadIdx.x + 256 * r] = MODE != 2 ? act_apply(rv[r], A.act) : rv[r];
      if (threadIdx.x < kTB) ab[2 * threadIdx.x] = ra, ab[2 * threadIdx.x + 1] = rb;
      __syncthreads();
      if (t0 + kTB < count) fetch(t0 + kTB, min(kTB, count - t0 - kTB));
      compute_round(nb);
      __syncthreads();
      reduce_round(t0, nb);
    }
  } else {
    for (int t0 = 0; t0 < count; t0 += kTB) {
      const int nb = min(kTB, count - t0);
      __syncthreads();   // the previous round's read-outs are out
      stage_rows(qg, A.ldq, first + t0, nb, d, dp, A.act, qs);
      if (MODE != 2) {
        stage_rows(kg, A.ldk, first + t0, nb, d, dp, A.act, ks);
        for (int i = threadIdx.x; i < nb * KC; i += blockDim.x) {
          const int j = i / KC, e = i - j * KC;
          const int64_t t = first + t0 + j;
          vs[i] = c0 + e < dv ? act_apply(A.v[t * A.ldv + (int64_t)h * dv + c0 + e], A.act) : 0.f;
        }
        for (int j = threadIdx.x; j < nb; j += blockDim.x) {
          const int64_t t = first + t0 + j;
          ab[2 * j] = A.a ? A.a[t * A.ld_ab + h] : A.a_head[h];
          ab[2 * j + 1] = A.b ? A.b[t * A.ld_ab + h] : 1.f;
        }
      }
      __syncthreads();
      compute_round(nb);
      __syncthreads();
      reduce_round(t0, nb);
    }
  }
  if (MODE != 2) {
#pragma unroll
    for (int cc = 0; cc < NC; ++cc) {
      const int c = c0 + 32 * cc + lane;
#pragma unroll
      for (int r = 0; r < DR; ++r) {
        const int i = warp * DR + r;
        if (c < dv && i < d) srow[(int64_t)i * dv + c] = S[cc][r];
      }
    }
  }
}

// Second pass of the tiled form: every element of the state carries on its own through the tiles of its segment,
// start[k] = S, S = (product of tile k's decays) * S + local[k], from the slot's state (zeros at position 0) to the state
// the slot keeps.  One thread per (segment, head, element): loads of the next tiles do not wait for the chain.
__global__ void outer_recurrence_carry_kernel(RecArgs A, const int32_t* __restrict__ tile_first, const int32_t* __restrict__ tile_count) {
  const int64_t per = (int64_t)A.d * A.dv;
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= per) return;
  const int h = blockIdx.y, seg = blockIdx.z;
  const int k0 = A.seg_tile0[seg], nk = A.seg_tiles[seg];
  const int row0 = tile_first[k0];
  float* st = A.state + ((int64_t)A.slot[row0] * A.H + h) * per + e;
  float S = A.pos[row0] == 0 ? 0.f : *st;
  const float* __restrict__ loc = A.ws_local + ((int64_t)k0 * A.H + h) * per + e;
  float* __restrict__ start = A.ws_start + ((int64_t)k0 * A.H + h) * per + e;
  const int64_t hop = (int64_t)A.H * per;
  int k = 0;
  for (; k + 4 <= nk; k += 4) {
    float l[4], pe[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      l[u] = loc[(k + u) * hop];
      pe[u] = A.pcum[(int64_t)(tile_first[k0 + k + u] + tile_count[k0 + k + u] - 1) * A.H + h];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      start[(k + u) * hop] = S;
      S = fmaf(pe[u], S, l[u]);
    }
  }
  for (; k < nk; ++k) {
    const float l = loc[k * hop], pe = A.pcum[(int64_t)(tile_first[k0 + k] + tile_count[k0 + k] - 1) * A.H + h];
    start[k * hop] = S;
    S = fmaf(pe, S, l);
  }
  *st = S;
}

// rows of the state per warp for a key size: 8 warps up to d = 256, more warps beyond
inline int rec_rows_per_warp(int d) { return d <= 32 ? 4 : d <= 64 ? 8 : d <= 128 ? 16 : 32; }
inline size_t rec_smem(int P, int DR, int KC) { return ((size_t)kTB * (2 * P * DR + KC + 2) + (size_t)P * kTB * KC) * sizeof(float); }

template <int DR, int MODE, int NC>
int launch_rec(const RecArgs& A, int n_ctas, cudaStream_t st) {
  constexpr int KC = 32 * NC;
  const int P = (A.d + DR - 1) / DR;
  const size_t smem = rec_smem(P, DR, KC);
  auto kern = outer_recurrence_kernel<DR, MODE, NC>;
  if (smem > 48 * 1024) {
    static bool set = false;   // per instantiation
    if (!set) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return AO_B200_ERR_CUDA;
      set = true;
    }
  }
  kern<<<dim3((unsigned)n_ctas, (unsigned)A.H, (unsigned)((A.dv + KC - 1) / KC)), P * 32, smem, st>>>(A);
  return lm_launch_status();
}

// two value columns per lane when the value size fills them (one pair of key / query loads then serves both); key sizes
// above 128 keep one column: their 32 rows per warp fill the registers
template <int MODE>
int launch_rec_mode(const RecArgs& A, int n_ctas, cudaStream_t st) {
  const bool two = A.dv > 32;
  switch (rec_rows_per_warp(A.d)) {
    case 4: return two ? launch_rec<4, MODE, 2>(A, n_ctas, st) : launch_rec<4, MODE, 1>(A, n_ctas, st);
    case 8: return two ? launch_rec<8, MODE, 2>(A, n_ctas, st) : launch_rec<8, MODE, 1>(A, n_ctas, st);
    case 16: return two ? launch_rec<16, MODE, 2>(A, n_ctas, st) : launch_rec<16, MODE, 1>(A, n_ctas, st);
    default: return launch_rec<32, MODE, 1>(A, n_ctas, st);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Input side of the state-space mixer.  One CTA per row: the convolution channels, then the heads' step sizes.
template <typename T>
__global__ void ssd_prep_kernel(const float* __restrict__ proj, int64_t ld, int64_t conv_off, int64_t dt_off, int64_t channels,
                                int taps, const T* __restrict__ conv_w, const T* __restrict__ conv_b,
                                const float* __restrict__ conv_state, const int32_t* __restrict__ slot,
                                const int32_t* __restrict__ pos, const int32_t* __restrict__ back, int H,
                                const T* __restrict__ dt_bias, const T* __restrict__ a_log, float* __restrict__ conv_out,
                                float* __restrict__ a_out, float* __restrict__ b_out) {
  const int64_t t = blockIdx.x;
  const int bk = back[t], p = pos[t];
  const float* st = conv_state + (int64_t)slot[t] * (taps > 1 ? taps - 1 : 1) * channels;
  for (int64_t c = threadIdx.x; c < channels; c += blockDim.x) {
    float acc = conv_b ? ldf(conv_b + c) : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int delta = taps - 1 - j;     // rows back in time
      float v = 0.f;
      if (delta <= bk)
        v = proj[(t - delta) * ld + conv_off + c];
      else if (delta <= p)
        v = st[(int64_t)(taps - 1 - (delta - bk)) * channels + c];
      acc = fmaf(ldf(conv_w + c * taps + j), v, acc);
    }
    conv_out[t * channels + c] = acc / (1.f + expf(-acc));
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float z = proj[t * ld + dt_off + h] + ldf(dt_bias + h);
    const float step = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));      // softplus, no clamp
    a_out[t * H + h] = expf(-expf(ldf(a_log + h)) * step);
    b_out[t * H + h] = step;
  }
}

// The last taps - 1 inputs of every sequence that the step touched become its convolution memory (oldest first); a
// segment shorter than that keeps the newest of what the memory held, and zeros stand in front of position 0.
__global__ void conv_state_save_kernel(const float* __restrict__ x, int64_t ldx, int64_t channels, int taps,
                                       const int32_t* __restrict__ slot, const int32_t* __restrict__ pos,
                                       const int32_t* __restrict__ back, const int32_t* __restrict__ ahead,
                                       float* __restrict__ state) {
  const int64_t t = blockIdx.x;
  if (ahead[t] != 0) return;
  const int keep = taps - 1, rows = back[t] + 1;
  const int64_t first = t - back[t];
  const int p0 = pos[t] - back[t];
  float* st = state + (int64_t)slot[t] * keep * channels;
  for (int64_t c = threadIdx.x; c < channels; c += blockDim.x) {
    for (int j = 0; j < keep; ++j) {      // ascending: a row of the old memory is read before it is overwritten
      const int s = rows - keep + j;      // index among the segment's rows
      float v = 0.f;
      if (s >= 0)
        v = x[(first + s) * ldx + c];
      else if (p0 + s >= 0)
        v = st[(int64_t)(keep + s) * channels + c];
      st[(int64_t)j * channels + c] = v;
    }
  }
}

// out = norm(y) * weight * sigmoid(gate)              (mode 0: the gate after the norm)
// out = norm(y * silu(gate)) * weight                 (mode 1: the gate in front of it)
// out = norm(y) * weight * silu(gate)                 (mode 2; weight == null: ones)
// with the norm taken over each of `groups` equal parts of the row.  grid (rows, groups).
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, int64_t ldy, const float* __restrict__ gate, int64_t ldg,
                                        int mode, int64_t width, int groups, const T* __restrict__ weight, float eps,
                                        T* __restrict__ out) {
  __shared__ float scratch[33];
  const int64_t t = blockIdx.x, per = width / groups, c0 = (int64_t)blockIdx.y * per;
  const float* yr = y + t * ldy + c0;
  const float* gr = gate + t * ldg + c0;
  float ss = 0.f;
  for (int64_t c = threadIdx.x; c < per; c += blockDim.x) {
    float v = yr[c];
    if (mode == 1) {
      const float z = gr[c];
      v *= z / (1.f + expf(-z));
    }
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float k = 1.f / sqrtf(ss / (float)per + eps);
  for (int64_t c = threadIdx.x; c < per; c += blockDim.x) {
    const float z = gr[c];
    float v = yr[c];
    const float wt = weight ? ldf(weight + c0 + c) : 1.f;
    if (mode == 1)
      v = v * (z / (1.f + expf(-z))) * k * wt;
    else if (mode == 2)
      v = v * k * wt * (z / (1.f + expf(-z)));
    else
      v = v * k * wt / (1.f + expf(-z));
    stf(out + t * width + c0 + c, v);
  }
}

// The same for small groups (a head's values): a warp per group, the group's values in registers between the sum of squares
// and the output.  grid (rows, ceil(groups / 8)), 8 warps.
constexpr int kGroupPerLane = 16;     // groups of up to 32 * 16 values
template <typename T>
__global__ void __launch_bounds__(256) gated_group_norm_warp_kernel(const float* __restrict__ y, int64_t ldy,
                                                                   const float* __restrict__ gate, int64_t ldg, int mode,
                                                                   int64_t width, int groups, const T* __restrict__ weight, float eps,
                                                                   T* __restrict__ out) {
  const int lane = threadIdx.x & 31, grp = blockIdx.y * 8 + (threadIdx.x >> 5);
  if (grp >= groups) return;
  const int64_t t = blockIdx.x;
  const int per = (int)(width / groups);
  const int64_t c0 = (int64_t)grp * per;
  const float* yr = y + t * ldy + c0;
  const float* gr = gate + t * ldg + c0;
  float v[kGroupPerLane], z[kGroupPerLane], ss = 0.f;
#pragma unroll
  for (int e = 0; e < kGroupPerLane; ++e) {
    const int c = lane + 32 * e;
    v[e] = c < per ? yr[c] : 0.f;
    z[e] = c < per ? gr[c] : 0.f;
    if (mode == 1) v[e] *= z[e] / (1.f + expf(-z[e]));
    ss = fmaf(v[e], v[e], ss);
  }
  const float k = 1.f / sqrtf(warp_sum(ss) / (float)per + eps);
#pragma unroll
  for (int e = 0; e < kGroupPerLane; ++e) {
    const int c = lane + 32 * e;
    if (c >= per) continue;
    const float wt = weight ? ldf(weight + c0 + c) : 1.f;
    float r = v[e] * k * wt;
    if (mode == 2)
      r *= z[e] / (1.f + expf(-z[e]));
    else if (mode == 0)
      r /= 1.f + expf(-z[e]);
    stf(out + t * width + c0 + c, r);
  }
}

}  // namespace

extern "C" int64_t ao_lm_outer_recurrence_workspace_bytes(int n_tiles, int64_t n, int H, int d, int dv) {
  return ((int64_t)2 * n_tiles * H * d * dv + n * H) * 4;
}

extern "C" int ao_lm_outer_recurrence(const float* q, int64_t ldq, const float* k, int64_t ldk, const float* v, int64_t ldv,
                                      int act, const float* a, const float* b, int64_t ld_ab, const float* a_head,
                                      const float* skip, int H, int G, int d, int dv, float* state, const int32_t* slot,
                                      const int32_t* pos, const int32_t* seg_first, const int32_t* seg_count, int n_segments,
                                      const int32_t* seg_tile0, const int32_t* seg_tiles, int n_whole_segments, int64_t n,
                                      float* workspace, float* out, int64_t ld_out, void* stream) {
  LM_CHECK_ARG(q && k && v && state && slot && pos && seg_first && seg_count && out && (a || a_head) && (!b || a));
  LM_CHECK_ARG(n_segments > 0 && H > 0 && G > 0 && H % G == 0 && H <= 65535 && d > 0 && dv > 0 && (act == 0 || act == 1));
  if (d > 1024) return AO_B200_ERR_UNSUPPORTED;
  RecArgs A{q, k, v, ldq, ldk, ldv, act, a, b, ld_ab, a_head, skip, H, G, d, dv, state, slot, pos, seg_first, seg_count, out, ld_out,
            nullptr, nullptr, nullptr, seg_tile0, seg_tiles};
  const cudaStream_t st = lm_stream(stream);
  if (!seg_tile0) return launch_rec_mode<0>(A, n_segments, st);
  // tiled form: seg_first / seg_count are tiles, segment s owns tiles seg_tile0[s] .. + seg_tiles[s] - 1
  LM_CHECK_ARG(seg_tiles && workspace && n_whole_segments > 0 && n_whole_segments <= 65535 && n > 0);
  const int64_t per = (int64_t)n_segments * H * d * dv;
  A.ws_local = workspace, A.ws_start = workspace + per, A.pcum = workspace + 2 * per;
  int rc = launch_rec_mode<1>(A, n_segments, st);
  if (rc != AO_B200_OK) return rc;
  outer_recurrence_carry_kernel<<<dim3((unsigned)(((int64_t)d * dv + 255) / 256), (unsigned)H, (unsigned)n_whole_segments), 256, 0, st>>>(
      A, seg_first, seg_count);
  rc = lm_launch_status();
  if (rc != AO_B200_OK) return rc;
  return launch_rec_mode<2>(A, n_segments, st);
}

extern "C" int ao_lm_ssd_prep(const float* proj, int64_t ld, int64_t conv_off, int64_t dt_off, int64_t n, int64_t channels,
                              int taps, const void* conv_w, const void* conv_b, int dt, const float* conv_state,
                              const int32_t* slot, const int32_t* pos, const int32_t* back, int H, const void* dt_bias,
                              const void* a_log, float* conv_out, float* a_out, float* b_out, void* stream) {
  LM_CHECK_ARG(proj && conv_w && conv_state && slot && pos && back && dt_bias && a_log && conv_out && a_out && b_out);
  LM_CHECK_ARG(n > 0 && channels > 0 && taps >= 1 && H > 0);
  LM_DISPATCH(dt, ssd_prep_kernel<T><<<(unsigned)n, 256, 0, lm_stream(stream)>>>(
                      proj, ld, conv_off, dt_off, channels, taps, static_cast<const T*>(conv_w), static_cast<const T*>(conv_b),
                      conv_state, slot, pos, back, H, static_cast<const T*>(dt_bias), static_cast<const T*>(a_log), conv_out, a_out,
                      b_out));
  return lm_launch_status();
}

extern "C" int ao_lm_conv_state_save(const float* x, int64_t ldx, int64_t n, int64_t channels, int taps, const int32_t* slot,
                                     const int32_t* pos, const int32_t* back, const int32_t* ahead, float* state, void* stream) {
  LM_CHECK_ARG(x && slot && pos && back && ahead && state && n > 0 && channels > 0 && taps >= 1);
  if (taps == 1) return AO_B200_OK;   // a one-tap convolution remembers nothing
  conv_state_save_kernel<<<(unsigned)n, 256, 0, lm_stream(stream)>>>(x, ldx, channels, taps, slot, pos, back, ahead, state);
  return lm_launch_status();
}

extern "C" int ao_lm_gated_group_norm(const float* y, int64_t ldy, const float* gate, int64_t ldg, int mode, int64_t n,
                                      int64_t width, int groups, const void* weight, int dt, float eps, void* out, void* stream) {
  LM_CHECK_ARG(y && gate && out && n > 0 && width > 0 && groups > 0 && groups <= 65535 && width % groups == 0);
  LM_CHECK_ARG(mode == 0 || mode == 1 || mode == 2);
  if (groups > 1 && width / groups <= 32 * kGroupPerLane) {
    LM_DISPATCH(dt, gated_group_norm_warp_kernel<T><<<dim3((unsigned)n, (unsigned)((groups + 7) / 8)), 256, 0, lm_stream(stream)>>>(
                        y, ldy, gate, ldg, mode, width, groups, static_cast<const T*>(weight), eps, static_cast<T*>(out)));
    return lm_launch_status();
  }
  LM_DISPATCH(dt, gated_group_norm_kernel<T><<<dim3((unsigned)n, (unsigned)groups), 256, 0, lm_stream(stream)>>>(
                      y, ldy, gate, ldg, mode, width, groups, static_cast<const T*>(weight), eps, static_cast<T*>(out)));
  return lm_launch_status();
}
