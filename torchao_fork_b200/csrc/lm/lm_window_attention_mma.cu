// Attention under a sliding window that keeps the first tokens, for prompt portions, on the tensor cores (bf16 storage):
// the same computation as ao_lm_window_attention — keys from the ring, the first-token store and the step's own rows; one or
// two softmax maps per head over the same values, a_1 - lambda a_2; unit RMS; a constant — for tiles of 64 consecutive rows
// of one sequence x one query head, with 64-key tiles shared by the 64 rows.
//
// mma.sync m16n8k16 with fp32 accumulators.  What the design computes in 32 bits stays in 32 bits:
//   scores   queries and keys are bf16 operands (the keys as the cache stores them), their products accumulate in fp32;
//            scale, maximum and exponential are fp32;
//   weights  exp(s - max) in fp32, multiplied into the values as THREE bf16 parts (p = p1 + p2 + p3 exactly, 24 bits),
//            the denominator summed in fp32 from the unsplit weights;
//   the maps' difference, the norm and the constant in fp32.
// The maps run one after the other over the same key tiles (the values come from L2 the second time); the first map's
// normalised result waits in shared memory, each thread's own elements, for the second.
// 4 warps x 16 rows.  K and V tiles arrive by cp.async in separate groups: the next keys load while the weights meet the
// values, the next values during the score product.
#include "lm_mma.cuh"

using namespace lm;

namespace {

constexpr int kPM = 64;      // query rows per CTA
constexpr int kPN = 64;      // keys per tile
constexpr int kPWarps = 4;
constexpr int kPad = 8;      // bf16 elements added to every shared-memory row: 16-byte rows land on distinct banks

struct WinPromptArgs {
  const float* qn;                         // [n][H][NM][d] fp32
  const __nv_bfloat16 *kn, *vn;            // step rows [n][G][NM][d], [n][G][dv]
  const __nv_bfloat16 *ring_k, *ring_v;    // [slots][ring][G][NM d], [slots][ring][G][dv]
  const __nv_bfloat16 *first_k, *first_v;  // [slots][first_rows][...]
  int ring, first_rows;
  const int32_t *slot, *pos, *back, *tile_first, *tile_count;
  int H, G, d, window, keep;
  float scale, lambda, out_scale, eps;
  int unit_rms;
  __nv_bfloat16* out;
  int64_t ld_out;
};

template <int NV, int NM>   // value size = 16 NV; maps per head
__global__ void __launch_bounds__(kPWarps * 32) window_attention_prompt_kernel(WinPromptArgs a) {
  using T = __nv_bfloat16;
  constexpr int DV = 16 * NV;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int d = a.d, G = a.G, KD = NM * d;
  const int QP = d + kPad, KP = d + kPad, VP = DV + kPad;
  T* Qs = reinterpret_cast<T*>(smem_raw);   // [NM][kPM][QP]
  T* Ks = Qs + (size_t)NM * kPM * QP;       // [kPN][KP]
  T* Vs = Ks + (size_t)kPN * KP;            // [kPN][VP]
  float* Os = reinterpret_cast<float*>(Vs + (size_t)kPN * VP);   // [kPM][DV], two maps only
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g4 = lane >> 2, t4 = lane & 3;
  const int h = blockIdx.y, g = h / (a.H / G);
  const int tile = gridDim.x - 1 - blockIdx.x;     // late tiles have the most keys: they start first
  const int first = a.tile_first[tile], count = min(a.tile_count[tile], kPM);
  const int pa = a.pos[first], back0 = a.back[first];
  const int p0 = pa - back0;                       // the first position the step brings of this sequence
  const int64_t seg_row0 = first - back0;
  const int lo = max(0, pa - a.window + 1);        // the oldest key of the first row's window
  const int nf = min(a.keep, lo);                  // kept first positions that lie in front of it
  const int nk = nf + (pa + count - lo);           // key index kk: the kept ones, then lo .. the last row's own position
  const int64_t s = a.slot[first];
  const T* ring_k = a.ring_k + (s * a.ring * G + g) * KD;
  const T* ring_v = a.ring_v + (s * a.ring * G + g) * DV;
  const T* first_k = a.first_k + (s * a.first_rows * G + g) * KD;
  const T* first_v = a.first_v + (s * a.first_rows * G + g) * DV;
  const T* step_k = a.kn + (seg_row0 * G + g) * KD;
  const T* step_v = a.vn + (seg_row0 * G + g) * DV;
  const int kc = d / 8;            // 16-byte chunks of a key row
  constexpr int vc = DV / 8;
  auto key_pos = [&](int kk) { return kk < nf ? kk : lo + (kk - nf); };

  auto load_k = [&](int k0, int m) {
    for (int i = threadIdx.x; i < kPN * kc; i += kPWarps * 32) {
      const int jj = i / kc, c = i - jj * kc, kk = k0 + jj;
      T* dst = Ks + (size_t)jj * KP + c * 8;
      if (kk < nk) {
        const int j = key_pos(kk);
        const T* src = j >= p0 ? step_k + (int64_t)(j - p0) * G * KD
                               : (j < a.first_rows ? first_k + (int64_t)j * G * KD : ring_k + (int64_t)(j % a.ring) * G * KD);
        cp_async16(dst, src + m * d + c * 8);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  auto load_v = [&](int k0) {
    for (int i = threadIdx.x; i < kPN * vc; i += kPWarps * 32) {
      const int jj = i / vc, c = i - jj * vc, kk = k0 + jj;
      T* dst = Vs + (size_t)jj * VP + c * 8;
      if (kk < nk) {
        const int j = key_pos(kk);
        const T* src = j >= p0 ? step_v + (int64_t)(j - p0) * G * DV
                               : (j < a.first_rows ? first_v + (int64_t)j * G * DV : ring_v + (int64_t)(j % a.ring) * G * DV);
        cp_async16(dst, src + c * 8);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  load_k(0, 0);
  cp_async_commit();
  load_v(0);
  cp_async_commit();
  // the query tiles of all maps as bf16 operands (rows past the run are zero)
  for (int i = threadIdx.x; i < NM * kPM * (d / 4); i += kPWarps * 32) {
    const int m = i / (kPM * (d / 4)), rem = i - m * (kPM * (d / 4));
    const int r = rem / (d / 4), c = (rem - r * (d / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < count) v = *reinterpret_cast<const float4*>(a.qn + (((int64_t)(first + r) * a.H + h) * NM + m) * d + c);
    *reinterpret_cast<uint2*>(Qs + ((size_t)m * kPM + r) * QP + c) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
  }
  const int r0 = warp * 16 + g4, r1 = r0 + 8;
  const int i0 = r0 < count ? pa + r0 : -1, i1 = r1 < count ? pa + r1 : -1;   // the rows' own positions (-1: no row)
  // ldmatrix row addresses of this lane: A (queries), B (keys), B transposed (values)
  const T* qa_ptr = Qs + (size_t)(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * QP + (lane >> 4) * 8;
  const T* kb_ptr = Ks + (size_t)((lane & 7) + (lane >> 4) * 8) * KP + ((lane >> 3) & 1) * 8;
  const T* vb_ptr = Vs + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * VP + (lane >> 4) * 8;
  const int ks_n = d / 16;
  // a warp skips a key tile that lies wholly in its rows' future, or wholly behind the window of its first row
  const int warp_rows = min(count, warp * 16 + 16) - warp * 16;      // <= 0: the warp has no rows
  const int w_lo = pa + warp * 16, w_hi = w_lo + warp_rows - 1;

#pragma unroll 1
  for (int m = 0; m < NM; ++m) {
    float o[2 * NV][4];
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows r0 and r1 (l: this thread's share)
    for (int k0 = 0; k0 < nk; k0 += kPN) {
      cp_async_wait<1>();
      __syncthreads();   // keys of this tile (and, the first time, the queries) are in shared memory
      float sc[kPN / 8][4];
#pragma unroll
      for (int i = 0; i < kPN / 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
      const int j_lo = key_pos(k0), j_hi = key_pos(min(k0 + kPN, nk) - 1);
      const bool live = warp_rows > 0 && j_lo <= w_hi && !(k0 >= nf && j_hi <= w_lo - a.window && j_lo >= a.keep);
      if (live) {
        for (int kk = 0; kk < ks_n; ++kk) {
          uint32_t qa[4];
          ldsm_x4(qa, qa_ptr + (size_t)m * kPM * QP + kk * 16);
#pragma unroll
          for (int j = 0; j < kPN / 16; ++j) {
            uint32_t b[4];
            ldsm_x4(b, kb_ptr + (size_t)j * 16 * KP + kk * 16);
            mma_bf16(sc[2 * j], qa, b[0], b[1]);
            mma_bf16(sc[2 * j + 1], qa, b[2], b[3]);
          }
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int i = 0; i < kPN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kk = k0 + i * 8 + 2 * t4 + e;
          const int j = key_pos(kk);
          const bool in = kk < nk;
          const bool s0 = in && j <= i0 && (i0 - j < a.window || j < a.keep);
          const bool s1 = in && j <= i1 && (i1 - j < a.window || j < a.keep);
          const float v0 = s0 ? sc[i][e] * a.scale : -INFINITY, v1 = s1 ? sc[i][2 + e] * a.scale : -INFINITY;
          sc[i][e] = v0, sc[i][2 + e] = v1;
          mx0 = fmaxf(mx0, v0);
          mx1 = fmaxf(mx1, v1);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
      const float c0 = n0 == -INFINITY ? 1.f : __expf(m0 - n0), c1 = n1 == -INFINITY ? 1.f : __expf(m1 - n1);
      m0 = n0, m1 = n1;
      l0 *= c0, l1 *= c1;
#pragma unroll
      for (int i = 0; i < 2 * NV; ++i) o[i][0] *= c0, o[i][1] *= c0, o[i][2] *= c1, o[i][3] *= c1;
#pragma unroll
      for (int i = 0; i < kPN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          sc[i][e] = n0 == -INFINITY ? 0.f : __expf(sc[i][e] - n0);
          sc[i][2 + e] = n1 == -INFINITY ? 0.f : __expf(sc[i][2 + e] - n1);
          l0 += sc[i][e];
          l1 += sc[i][2 + e];
        }
      }
      cp_async_wait<0>();
      __syncthreads();   // values of this tile are in shared memory, and every warp is done with its keys
      const bool more = k0 + kPN < nk;
      if (more) load_k(k0 + kPN, m);   // lands while the weights meet the values
      else if (m + 1 < NM) load_k(0, m + 1);
      cp_async_commit();
      if (live) {
        // the three bf16 parts of the weights as A fragments; every value fragment is loaded once and meets all three
        uint32_t pw[3][kPN / 16][4];
#pragma unroll
        for (int part = 0; part < 3; ++part) {
#pragma unroll
          for (int j = 0; j < kPN / 16; ++j) {
            const float h00 = split_bf16(sc[2 * j][0]), h01 = split_bf16(sc[2 * j][1]);
            const float h10 = split_bf16(sc[2 * j][2]), h11 = split_bf16(sc[2 * j][3]);
            const float h20 = split_bf16(sc[2 * j + 1][0]), h21 = split_bf16(sc[2 * j + 1][1]);
            const float h30 = split_bf16(sc[2 * j + 1][2]), h31 = split_bf16(sc[2 * j + 1][3]);
            pw[part][j][0] = pack_bf16(h00, h01);
            pw[part][j][1] = pack_bf16(h10, h11);
            pw[part][j][2] = pack_bf16(h20, h21);
            pw[part][j][3] = pack_bf16(h30, h31);
          }
        }
#pragma unroll
        for (int j = 0; j < kPN / 16; ++j) {
#pragma unroll
          for (int v0 = 0; v0 < NV; v0 += 4) {   // four fragments at a time: eight accumulators between two uses of one
            uint32_t b[4][4];
#pragma unroll
            for (int vv = 0; vv < 4; ++vv)
              if (v0 + vv < NV) ldsm_x4_trans(b[vv], vb_ptr + (size_t)j * 16 * VP + (v0 + vv) * 16);
#pragma unroll
            for (int part = 0; part < 3; ++part) {
#pragma unroll
              for (int vv = 0; vv < 4; ++vv) {
                if (v0 + vv < NV) {
                  mma_bf16(o[2 * (v0 + vv)], pw[part][j], b[vv][0], b[vv][1]);
                  mma_bf16(o[2 * (v0 + vv) + 1], pw[part][j], b[vv][2], b[vv][3]);
                }
              }
            }
          }
        }
      }
      __syncthreads();   // every warp is done with this tile's values
      if (more) load_v(k0 + kPN);   // lands during the next tile's score product
      else if (m + 1 < NM) load_v(0);
      cp_async_commit();
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float k0n = i0 >= 0 ? 1.f / l0 : 0.f, k1n = i1 >= 0 ? 1.f / l1 : 0.f;
    if (m + 1 < NM) {   // the first map's result waits, element by element, with the thread that made it
#pragma unroll
      for (int i = 0; i < 2 * NV; ++i) {
        float* p0_ = Os + (size_t)r0 * DV + i * 8 + 2 * t4;
        float* p1_ = Os + (size_t)r1 * DV + i * 8 + 2 * t4;
        p0_[0] = o[i][0] * k0n, p0_[1] = o[i][1] * k0n;
        p1_[0] = o[i][2] * k1n, p1_[1] = o[i][3] * k1n;
      }
      continue;
    }
    float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i) {
      o[i][0] *= k0n, o[i][1] *= k0n, o[i][2] *= k1n, o[i][3] *= k1n;
      if (NM == 2) {
        const float* p0_ = Os + (size_t)r0 * DV + i * 8 + 2 * t4;
        const float* p1_ = Os + (size_t)r1 * DV + i * 8 + 2 * t4;
        o[i][0] = p0_[0] - a.lambda * o[i][0], o[i][1] = p0_[1] - a.lambda * o[i][1];
        o[i][2] = p1_[0] - a.lambda * o[i][2], o[i][3] = p1_[1] - a.lambda * o[i][3];
      }
      ss0 = fmaf(o[i][0], o[i][0], fmaf(o[i][1], o[i][1], ss0));
      ss1 = fmaf(o[i][2], o[i][2], fmaf(o[i][3], o[i][3], ss1));
    }
    ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1);
    ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
    ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1);
    ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
    const bool pair_store = a.ld_out % 2 == 0;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = half ? r1 : r0;
      if (r >= count) continue;
      float k = a.out_scale;
      if (a.unit_rms) k /= sqrtf((half ? ss1 : ss0) / (float)DV + a.eps);
      T* dst = a.out + (int64_t)(first + r) * a.ld_out + (int64_t)h * DV + 2 * t4;
#pragma unroll
      for (int i = 0; i < 2 * NV; ++i) {
        const float y0 = o[i][2 * half] * k, y1 = o[i][2 * half + 1] * k;
        if (pair_store) {
          *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(y0, y1);
        } else {   // rows of odd length: every other row starts on an odd element
          dst[i * 8] = __float2bfloat16_rn(y0);
          dst[i * 8 + 1] = __float2bfloat16_rn(y1);
        }
      }
    }
  }
  cp_async_wait<0>();
}

inline size_t win_prompt_smem(int nm, int d, int dv) {
  return ((size_t)nm * kPM * (d + kPad) + (size_t)kPN * (d + kPad) + (size_t)kPN * (dv + kPad)) * 2 +
         (nm == 2 ? (size_t)kPM * dv * 4 : 0);
}

inline bool win_prompt_ok(int dt, int nm, int H, int G, int d, int dv) {
  if (dt != AO_LM_BF16 || (nm != 1 && nm != 2) || G <= 0 || H % G || d <= 0 || d % 16 || dv % 16 || dv < 16 || dv > 128) return false;
  return win_prompt_smem(nm, d, dv) <= 200 * 1024;
}

template <int NV, int NM>
int launch_win_prompt(const WinPromptArgs& a, int n_tiles, cudaStream_t st) {
  const size_t smem = win_prompt_smem(NM, a.d, 16 * NV);
  auto kern = window_attention_prompt_kernel<NV, NM>;
  if (smem > 48 * 1024) {
    static bool set = false;   // per instantiation
    if (!set) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return AO_B200_ERR_CUDA;
      set = true;
    }
  }
  kern<<<dim3((unsigned)n_tiles, (unsigned)a.H), kPWarps * 32, smem, st>>>(a);
  return lm_launch_status();
}

}  // namespace

extern "C" int ao_lm_window_attention_prompt_plan(int dt, int n_maps, int H, int G, int d, int dv, int* tile_rows) {
  LM_CHECK_ARG(tile_rows);
  *tile_rows = win_prompt_ok(dt, n_maps, H, G, d, dv) ? kPM : 0;
  return AO_B200_OK;
}

extern "C" int ao_lm_window_attention_prompt(const float* qn, const void* kn, const void* vn, const void* ring_k, const void* ring_v,
                                             const void* first_k, const void* first_v, int ring, int first_rows, int dt,
                                             const int32_t* slot, const int32_t* pos, const int32_t* back,
                                             const int32_t* tile_first, const int32_t* tile_count, int n_tiles, int n_maps, int H,
                                             int G, int d, int dv, int window, int keep, float scale, float lambda, int unit_rms,
                                             float eps, float out_scale, void* out, int64_t ld_out, void* stream) {
  LM_CHECK_ARG(qn && kn && vn && ring_k && ring_v && slot && pos && back && tile_first && tile_count && out);
  LM_CHECK_ARG(n_tiles > 0 && window > 0 && keep >= 0 && ring >= window && first_rows >= keep && (first_rows == 0 || (first_k && first_v)));
  LM_CHECK_ARG(H > 0 && H <= 65535);
  if (!win_prompt_ok(dt, n_maps, H, G, d, dv)) return AO_B200_ERR_UNSUPPORTED;
  // 16-byte copies of queries, keys and values; the result is stored in pairs when its rows allow it
  LM_CHECK_ARG(reinterpret_cast<uintptr_t>(out) % 4 == 0 && reinterpret_cast<uintptr_t>(qn) % 16 == 0 &&
               reinterpret_cast<uintptr_t>(kn) % 16 == 0 && reinterpret_cast<uintptr_t>(vn) % 16 == 0 &&
               reinterpret_cast<uintptr_t>(ring_k) % 16 == 0 && reinterpret_cast<uintptr_t>(ring_v) % 16 == 0 &&
               reinterpret_cast<uintptr_t>(first_k) % 16 == 0 && reinterpret_cast<uintptr_t>(first_v) % 16 == 0);
  using T = __nv_bfloat16;
  WinPromptArgs a{qn, static_cast<const T*>(kn), static_cast<const T*>(vn), static_cast<const T*>(ring_k),
                  static_cast<const T*>(ring_v), static_cast<const T*>(first_k ? first_k : ring_k),
                  static_cast<const T*>(first_v ? first_v : ring_v), ring, first_rows, slot, pos, back, tile_first, tile_count,
                  H, G, d, window, keep, scale, lambda, out_scale, eps, unit_rms, static_cast<T*>(out), ld_out};
  const cudaStream_t st = lm_stream(stream);
#define LM_WP(NV)                                                    \
  case NV:                                                           \
    return n_maps == 2 ? launch_win_prompt<NV, 2>(a, n_tiles, st) : launch_win_prompt<NV, 1>(a, n_tiles, st);
  switch (dv / 16) { LM_WP(1) LM_WP(2) LM_WP(3) LM_WP(4) LM_WP(5) LM_WP(6) LM_WP(7) LM_WP(8) }
#undef LM_WP
  return AO_B200_ERR_UNSUPPORTED;
}
