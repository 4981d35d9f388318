// Matrix-state recurrence with a decay per key channel and a bonus for the current token (time mixing in the RWKV manner):
//     o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t,        S_t = diag(w_t) S_(t-1) + k_t v_t^T          (S: d x dv per head)
// with w_t either given, or made on load from the pre-activation z as w = exp(-exp(z + bias)).  The state lives in fp32
// [slots][H][d][dv] and is carried from step to step; a sequence that starts at position 0 starts from zeros without
// reading its slot.  Every product and sum is fp32, and a token is folded into the state by the same instructions whether
// it arrives alone or inside a prompt portion.
//
// One CTA = one segment (consecutive rows of one sequence) x one head x 32 value columns: lane = column, warp p owns DR key
// channels of the state in registers; rows are staged kTB at a time in shared memory, every warp leaves its partial
// read-outs there and the block adds them up once per round.  A segment longer than a tile runs in three launches:
// every tile from a zero state (keeping, per row, the product of the decays of the tile's rows in front of it), the
// tiles' start states carried through the segment element by element, and the read-out of each tile's start state,
// decayed up to each row, added to the rows.  No quotient of decay products is ever formed.
//
// The kernel that ends a segment also stores the row that a token-shift layer must remember (`shift_src`).
#include "lm_common.cuh"

using namespace lm;

namespace {

constexpr int kTB = 16;
constexpr int kWarps = 8;

struct ChanArgs {
  const float *r, *k, *v;          // rows [n][ld*], H heads of d (r, k) and dv (v)
  int64_t ldr, ldk, ldv;
  const float* w;                  // [n][ldw] per (row, head, channel): the decay, or its pre-activation
  int64_t ldw;
  const void* w_bias;              // storage type [H d]; non-null: w = exp(-exp(w + bias))
  const void* bonus;               // storage type [H d]; null: none
  int H, d, dv;
  float* state;                    // [slots][H][d][dv]
  const int32_t *slot, *pos, *seg_first, *seg_count;
  float* out;                      // [n][ld_out]
  int64_t ld_out;
  float *ws_local, *ws_start, *pcum, *ptot;   // tiled form
  const int32_t *seg_tile0, *seg_tiles;
  const float* shift_src;          // [n][shift_width]; the segment's last row goes to shift_state[slot]
  float* shift_state;
  int64_t shift_width;
};

template <typename T>
__device__ __forceinline__ float decay_of(const ChanArgs& A, int64_t t, int h, int c) {
  const float z = A.w[t * A.ldw + (int64_t)h * A.d + c];
  return A.w_bias ? expf(-expf(z + ldf(static_cast<const T*>(A.w_bias) + (int64_t)h * A.d + c))) : z;
}

// MODE 0: whole segments on the slots' state.  MODE 1: a tile from a zero state (its final state -> ws_local, per row the
// product of the decays in front of it -> pcum, the product over the whole tile -> ptot).  MODE 2: out += read-out of the
// tile's start state (ws_start) decayed up to each row.
template <typename T, int DR, int MODE>
__global__ void __launch_bounds__(kWarps * 32) channel_recurrence_kernel(ChanArgs A) {
  constexpr int DP = kWarps * DR;
  __shared__ __align__(16) float rs[kTB][DP], ks[kTB][DP], wsh[kTB][DP], vs[kTB][32], op[kWarps][kTB][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seg = blockIdx.x, h = blockIdx.y, c = blockIdx.z * 32 + lane;
  const int first = A.seg_first[seg], count = A.seg_count[seg];
  const int d = A.d, dv = A.dv;
  float* srow = MODE == 0 ? A.state + (((int64_t)A.slot[first] * A.H + h) * d) * dv
                          : (MODE == 1 ? A.ws_local : A.ws_start) + (((int64_t)seg * A.H + h) * d) * dv;
  const bool fresh = MODE == 1 || (MODE == 0 && A.pos[first] == 0);
  float S[DR], ub[DR];
#pragma unroll
  for (int i = 0; i < DR; ++i) {
    const int ch = warp * DR + i;
    S[i] = (!fresh && c < dv && ch < d) ? srow[(int64_t)ch * dv + c] : 0.f;
    ub[i] = (MODE != 2 && A.bonus && ch < d) ? ldf(static_cast<const T*>(A.bonus) + (int64_t)h * d + ch) : 0.f;
  }
  // MODE 1: the decays' running products, once per (tile, head): thread ch follows its channel through the staged rows
  const bool products = MODE == 1 && blockIdx.z == 0 && (int)threadIdx.x < d;
  float run = 1.f;
  if (MODE == 0 && A.shift_state && h == 0 && blockIdx.z == 0) {
    const float* src = A.shift_src + (int64_t)(first + count - 1) * A.shift_width;
    float* dst = A.shift_state + (int64_t)A.slot[first] * A.shift_width;
    for (int64_t i = threadIdx.x; i < A.shift_width; i += blockDim.x) dst[i] = src[i];
  }
  for (int t0 = 0; t0 < count; t0 += kTB) {
    const int nb = min(kTB, count - t0);
    __syncthreads();   // the previous round's read-outs are out
    for (int i = threadIdx.x; i < nb * DP; i += blockDim.x) {
      const int j = i / DP, ch = i - j * DP;
      const int64_t t = first + t0 + j;
      const bool in = ch < d;
      rs[j][ch] = in ? A.r[t * A.ldr + (int64_t)h * d + ch] : 0.f;
      if (MODE != 2) {
        ks[j][ch] = in ? A.k[t * A.ldk + (int64_t)h * d + ch] : 0.f;
        wsh[j][ch] = in ? decay_of<T>(A, t, h, ch) : 1.f;
      } else {
        wsh[j][ch] = in ? A.pcum[(t * A.H + h) * d + ch] : 0.f;
      }
    }
    if (MODE != 2)
      for (int i = threadIdx.x; i < nb * 32; i += blockDim.x) {
        const int j = i >> 5, e = i & 31, cc = blockIdx.z * 32 + e;
        vs[j][e] = cc < dv ? A.v[(int64_t)(first + t0 + j) * A.ldv + (int64_t)h * dv + cc] : 0.f;
      }
    __syncthreads();
    if (products) {
      for (int j = 0; j < nb; ++j) {
        A.pcum[((int64_t)(first + t0 + j) * A.H + h) * d + threadIdx.x] = run;
        run *= wsh[j][threadIdx.x];
      }
    }
    for (int j = 0; j < nb; ++j) {
      float o0 = 0.f, o1 = 0.f;
      if (MODE != 2) {
        const float vv = vs[j][lane];
#pragma unroll
        for (int i = 0; i < DR; i += 4) {      // four channels per 16-byte read of the staged rows
          const int ch = warp * DR + i;
          const float4 r4 = *reinterpret_cast<const float4*>(&rs[j][ch]), k4 = *reinterpret_cast<const float4*>(&ks[j][ch]);
          const float4 w4 = *reinterpret_cast<const float4*>(&wsh[j][ch]);
          const float kv0 = k4.x * vv, kv1 = k4.y * vv, kv2 = k4.z * vv, kv3 = k4.w * vv;
          o0 = fmaf(r4.x, fmaf(ub[i], kv0, S[i]), o0);
          o1 = fmaf(r4.y, fmaf(ub[i + 1], kv1, S[i + 1]), o1);
          o0 = fmaf(r4.z, fmaf(ub[i + 2], kv2, S[i + 2]), o0);
          o1 = fmaf(r4.w, fmaf(ub[i + 3], kv3, S[i + 3]), o1);
          S[i] = fmaf(w4.x, S[i], kv0);
          S[i + 1] = fmaf(w4.y, S[i + 1], kv1);
          S[i + 2] = fmaf(w4.z, S[i + 2], kv2);
          S[i + 3] = fmaf(w4.w, S[i + 3], kv3);
        }
      } else {
#pragma unroll
        for (int i = 0; i < DR; i += 4) {
          const int ch = warp * DR + i;
          const float4 r4 = *reinterpret_cast<const float4*>(&rs[j][ch]), w4 = *reinterpret_cast<const float4*>(&wsh[j][ch]);
          o0 = fmaf(r4.x * w4.x, S[i], o0);
          o1 = fmaf(r4.y * w4.y, S[i + 1], o1);
          o0 = fmaf(r4.z * w4.z, S[i + 2], o0);
          o1 = fmaf(r4.w * w4.w, S[i + 3], o1);
        }
      }
      op[warp][j][lane] = o0 + o1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nb * 32; i += blockDim.x) {
      const int j = i >> 5, e = i & 31, cc = blockIdx.z * 32 + e;
      if (cc >= dv) continue;
      float o = 0.f;
#pragma unroll
      for (int p = 0; p < kWarps; ++p) o += op[p][j][e];
      float* dst = A.out + (int64_t)(first + t0 + j) * A.ld_out + (int64_t)h * dv + cc;
      *dst = MODE == 2 ? *dst + o : o;
    }
  }
  if (products) A.ptot[((int64_t)seg * A.H + h) * d + threadIdx.x] = run;
  if (MODE != 2) {
#pragma unroll
    for (int i = 0; i < DR; ++i) {
      const int ch = warp * DR + i;
      if (c < dv && ch < d) srow[(int64_t)ch * dv + c] = S[i];
    }
  }
}

// Second pass of the tiled form: every element of the state carries on its own through the tiles of its segment,
// start[k] = S, S = (product of tile k's decays of its channel) * S + local[k].
__global__ void channel_recurrence_carry_kernel(ChanArgs A, const int32_t* __restrict__ tile_first,
                                                const int32_t* __restrict__ tile_count) {
  const int64_t per = (int64_t)A.d * A.dv;
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int h = blockIdx.y, seg = blockIdx.z;
  const int k0 = A.seg_tile0[seg], nk = A.seg_tiles[seg];
  const int row0 = tile_first[k0];
  if (A.shift_state && h == 0) {
    const int last = tile_first[k0 + nk - 1] + tile_count[k0 + nk - 1] - 1;
    if (e < A.shift_width) A.shift_state[(int64_t)A.slot[row0] * A.shift_width + e] = A.shift_src[(int64_t)last * A.shift_width + e];
  }
  if (e >= per) return;
  const int ch = (int)(e / A.dv);
  float* st = A.state + ((int64_t)A.slot[row0] * A.H + h) * per + e;
  float S = A.pos[row0] == 0 ? 0.f : *st;
  const int64_t hop = (int64_t)A.H * per;
  const float* loc = A.ws_local + ((int64_t)k0 * A.H + h) * per + e;
  float* start = A.ws_start + ((int64_t)k0 * A.H + h) * per + e;
  for (int k = 0; k < nk; ++k) {
    start[k * hop] = S;
    S = fmaf(A.ptot[((int64_t)(k0 + k) * A.H + h) * A.d + ch], S, loc[k * hop]);
  }
  *st = S;
}

template <typename T, int MODE>
int launch_chan(const ChanArgs& A, int n_ctas, cudaStream_t st) {
  const dim3 grid((unsigned)n_ctas, (unsigned)A.H, (unsigned)((A.dv + 31) / 32));
  if (A.d <= 32) channel_recurrence_kernel<T, 4, MODE><<<grid, kWarps * 32, 0, st>>>(A);
  else if (A.d <= 64) channel_recurrence_kernel<T, 8, MODE><<<grid, kWarps * 32, 0, st>>>(A);
  else channel_recurrence_kernel<T, 16, MODE><<<grid, kWarps * 32, 0, st>>>(A);
  return lm_launch_status();
}

}  // namespace

extern "C" int64_t ao_lm_channel_recurrence_workspace_bytes(int n_tiles, int64_t n, int H, int d, int dv) {
  return ((int64_t)2 * n_tiles * H * d * dv + n * H * d + (int64_t)n_tiles * H * d) * 4;
}

extern "C" int ao_lm_channel_recurrence(const float* r, int64_t ldr, const float* k, int64_t ldk, const float* v, int64_t ldv,
                                        const float* w, int64_t ldw, const void* w_bias, const void* bonus, int dt, int H, int d,
                                        int dv, float* state, const int32_t* slot, const int32_t* pos, const int32_t* seg_first,
                                        const int32_t* seg_count, int n_segments, const int32_t* seg_tile0,
                                        const int32_t* seg_tiles, int n_whole_segments, int64_t n, float* workspace,
                                        const float* shift_src, float* shift_state, int64_t shift_width, float* out,
                                        int64_t ld_out, void* stream) {
  LM_CHECK_ARG(r && k && v && w && state && slot && pos && seg_first && seg_count && out);
  LM_CHECK_ARG(n_segments > 0 && H > 0 && H <= 65535 && d > 0 && dv > 0 && (!shift_state || (shift_src && shift_width > 0)));
  if (d > 128) return AO_B200_ERR_UNSUPPORTED;
  ChanArgs A{r, k, v, ldr, ldk, ldv, w, ldw, w_bias, bonus, H, d, dv, state, slot, pos, seg_first, seg_count, out, ld_out,
             nullptr, nullptr, nullptr, nullptr, seg_tile0, seg_tiles, shift_src, shift_state, shift_width};
  const cudaStream_t st = lm_stream(stream);
  if (!seg_tile0) {
    LM_DISPATCH(dt, return launch_chan<T, 0>(A, n_segments, st));
  }
  LM_CHECK_ARG(seg_tiles && workspace && n_whole_segments > 0 && n_whole_segments <= 65535 && n > 0);
  const int64_t per = (int64_t)n_segments * H * d * dv;
  A.ws_local = workspace, A.ws_start = workspace + per, A.pcum = workspace + 2 * per, A.ptot = A.pcum + n * H * d;
  int rc = AO_B200_OK;
  LM_DISPATCH(dt, rc = launch_chan<T, 1>(A, n_segments, st));
  if (rc != AO_B200_OK) return rc;
  const int64_t elems = (int64_t)d * dv > shift_width ? (int64_t)d * dv : (shift_state ? shift_width : (int64_t)d * dv);
  channel_recurrence_carry_kernel<<<dim3((unsigned)((elems + 255) / 256), (unsigned)H, (unsigned)n_whole_segments), 256, 0, st>>>(
      A, seg_first, seg_count);
  rc = lm_launch_status();
  if (rc != AO_B200_OK) return rc;
  LM_DISPATCH(dt, rc = launch_chan<T, 2>(A, n_segments, st));
  return rc;
}
