// Chunked attention for prompt portions on the tensor cores (bf16 storage): the same computation as
// ao_lm_chunk_attention — keys of the query's own chunk, from the ring and from the step's own rows; soft-capped scores
// plus a bias per distance and head; softmax; sigmoid gate — for tiles of 64 consecutive rows of one sequence inside one
// chunk x one query head, with 64-key tiles shared by the 64 rows.
//
// mma.sync m16n8k16 with fp32 accumulators.  What the design computes in 32 bits stays in 32 bits:
//   scores   the unit-RMS queries and keys are bf16 operands (the keys as the ring stores them), their products
//            accumulate in fp32; scale, soft cap, bias, maximum and exponential are fp32;
//   weights  exp(s - max) in fp32, multiplied into the values as THREE bf16 parts (p = p1 + p2 + p3 exactly, 24 bits),
//            the denominator summed in fp32 from the unsplit weights;
//   gate and normalisation in fp32.
// 4 warps x 16 rows.  K and V tiles arrive by cp.async in separate groups: the next keys load while the weights meet the
// values, the next values during the score product.
#include "lm_mma.cuh"

using namespace lm;

namespace {

constexpr int kPM = 64;      // query rows per CTA
constexpr int kPN = 64;      // keys per tile
constexpr int kPWarps = 4;
constexpr int kPad = 8;      // bf16 elements added to every shared-memory row: 16-byte rows land on distinct banks

// tanh through one exponential: 1 - 2 / (e^(2x) + 1).  Absolute error of a few 1e-7, which is far below what the bf16
// operands of this kernel leave in a score; the fp32 kernel keeps tanhf.
__device__ __forceinline__ float tanh_fast(float x) { return 1.f - __fdividef(2.f, __expf(2.f * x) + 1.f); }

struct PromptArgs {
  const float* qn;                       // [n][H][d] unit-RMS queries, fp32
  const __nv_bfloat16 *kn, *vn;          // step rows [n][G][d], [n][G][dv]
  const __nv_bfloat16 *ring_k, *ring_v;  // [slots][C][G][d], [slots][C][G][dv]
  const float* gate;
  int64_t ld_gate;
  const float* bias;                     // [H][n_dist]; null: none
  int n_dist;
  const float* sink;                     // [H]; null: none
  const int32_t *slot, *pos, *back, *tile_first, *tile_count;
  int H, G, d, C;
  float scale, softcap, out_scale;
  __nv_bfloat16* out;
  int64_t ld_out;
};

template <int NV>   // value size = 16 NV
__global__ void __launch_bounds__(kPWarps * 32) chunk_attention_prompt_kernel(PromptArgs a) {
  using T = __nv_bfloat16;
  constexpr int DV = 16 * NV;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int d = a.d, C = a.C, G = a.G;
  const int QP = d + kPad, KP = d + kPad, VP = DV + kPad;
  T* Qs = reinterpret_cast<T*>(smem_raw);   // [kPM][QP]
  T* Ks = Qs + (size_t)kPM * QP;            // [kPN][KP]
  T* Vs = Ks + (size_t)kPN * KP;            // [kPN][VP]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g4 = lane >> 2, t4 = lane & 3;
  const int h = blockIdx.y, g = h / (a.H / G);
  const int tile = gridDim.x - 1 - blockIdx.x;
  const int first = a.tile_first[tile], count = min(a.tile_count[tile], kPM);
  const int pos0 = a.pos[first], back0 = a.back[first];
  const int off0 = pos0 % C;                       // the first row's place in its chunk = its own key index
  const int n_ring = max(0, off0 - back0);         // keys of the chunk that earlier steps left in the ring
  const int64_t step_row0 = first - min(back0, off0);
  const int k_hi = off0 + count;                   // key indices 0 .. the last row's own
  const T* ring_k = a.ring_k + ((int64_t)a.slot[first] * C * G + g) * d;
  const T* ring_v = a.ring_v + ((int64_t)a.slot[first] * C * G + g) * DV;
  const T* step_k = a.kn + (step_row0 * G + g) * d;
  const T* step_v = a.vn + (step_row0 * G + g) * DV;
  const int kc = d / 8;            // 16-byte chunks of a key row
  constexpr int vc = DV / 8;

  auto load_k = [&](int k0) {
    for (int i = threadIdx.x; i < kPN * kc; i += kPWarps * 32) {
      const int j = i / kc, c = i - j * kc, key = k0 + j;
      T* dst = Ks + (size_t)j * KP + c * 8;
      if (key < k_hi)
        cp_async16(dst, (key < n_ring ? ring_k + (int64_t)key * G * d : step_k + (int64_t)(key - n_ring) * G * d) + c * 8);
      else
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
  };
  auto load_v = [&](int k0) {
    for (int i = threadIdx.x; i < kPN * vc; i += kPWarps * 32) {
      const int j = i / vc, c = i - j * vc, key = k0 + j;
      T* dst = Vs + (size_t)j * VP + c * 8;
      if (key < k_hi)
        cp_async16(dst, (key < n_ring ? ring_v + (int64_t)key * G * DV : step_v + (int64_t)(key - n_ring) * G * DV) + c * 8);
      else
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
  };
  load_k(0);
  cp_async_commit();
  load_v(0);
  cp_async_commit();
  // the query tile as bf16 operands (rows past the run are zero)
  for (int i = threadIdx.x; i < kPM * (d / 4); i += kPWarps * 32) {
    const int r = i / (d / 4), c = (i - r * (d / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < count) v = *reinterpret_cast<const float4*>(a.qn + ((int64_t)(first + r) * a.H + h) * d + c);
    *reinterpret_cast<uint2*>(Qs + (size_t)r * QP + c) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
  }
  float o[2 * NV][4];
#pragma unroll
  for (int i = 0; i < 2 * NV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows 16 warp + g4 and + 8 (l: this thread's share)
  const int r0 = warp * 16 + g4, r1 = r0 + 8;
  const int lim0 = r0 < count ? off0 + r0 : -1, lim1 = r1 < count ? off0 + r1 : -1;   // the rows' own key indices
  const float* bias = a.bias ? a.bias + (int64_t)h * a.n_dist : nullptr;
  const int nd1 = a.n_dist - 1;
  // ldmatrix row addresses of this lane: A (queries), B (keys), B transposed (values)
  const T* qa_ptr = Qs + (size_t)(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * QP + (lane >> 4) * 8;
  const T* kb_ptr = Ks + (size_t)((lane & 7) + (lane >> 4) * 8) * KP + ((lane >> 3) & 1) * 8;
  const T* vb_ptr = Vs + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * VP + (lane >> 4) * 8;
  const int ks_n = d / 16;
  // a warp whose rows all come before a key tile skips the tile (its weights there are all zero)
  const int warp_last = min(count, warp * 16 + 16) - 1;             // < warp * 16: the warp has no rows
  const int warp_hi = warp_last >= warp * 16 ? off0 + warp_last + 1 : 0;
  const float cap = a.softcap, inv_cap = cap > 0.f ? 1.f / cap : 0.f;

  for (int k0 = 0; k0 < k_hi; k0 += kPN) {
    cp_async_wait<1>();
    __syncthreads();   // keys of this tile (and, the first time, the queries) are in shared memory
    float s[kPN / 8][4];
#pragma unroll
    for (int i = 0; i < kPN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    const bool live = k0 < warp_hi;
    if (live) {
      for (int kk = 0; kk < ks_n; ++kk) {
        uint32_t qa[4];
        ldsm_x4(qa, qa_ptr + kk * 16);
#pragma unroll
        for (int j = 0; j < kPN / 16; ++j) {
          uint32_t b[4];
          ldsm_x4(b, kb_ptr + (size_t)j * 16 * KP + kk * 16);
          mma_bf16(s[2 * j], qa, b[0], b[1]);
          mma_bf16(s[2 * j + 1], qa, b[2], b[3]);
        }
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < kPN / 8; ++i) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = k0 + i * 8 + 2 * t4 + e;
        float v0 = -INFINITY, v1 = -INFINITY;
        if (key <= lim0) {
          v0 = s[i][e] * a.scale;
          if (cap > 0.f) v0 = cap * tanh_fast(v0 * inv_cap);
          if (bias) v0 += __ldg(bias + min(lim0 - key, nd1));
        }
        if (key <= lim1) {
          v1 = s[i][2 + e] * a.scale;
          if (cap > 0.f) v1 = cap * tanh_fast(v1 * inv_cap);
          if (bias) v1 += __ldg(bias + min(lim1 - key, nd1));
        }
        s[i][e] = v0, s[i][2 + e] = v1;
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
        s[i][e] = n0 == -INFINITY ? 0.f : __expf(s[i][e] - n0);
        s[i][2 + e] = n1 == -INFINITY ? 0.f : __expf(s[i][2 + e] - n1);
        l0 += s[i][e];
        l1 += s[i][2 + e];
      }
    }
    cp_async_wait<0>();
    __syncthreads();   // values of this tile are in shared memory, and every warp is done with its keys
    const bool more = k0 + kPN < k_hi;
    if (more) load_k(k0 + kPN);   // lands while the weights meet the values
    cp_async_commit();
    if (live) {
      // the three bf16 parts of the weights as A fragments; every value fragment is loaded once and meets all three
      uint32_t pa[3][kPN / 16][4];
#pragma unroll
      for (int part = 0; part < 3; ++part) {
#pragma unroll
        for (int j = 0; j < kPN / 16; ++j) {
          const float h00 = split_bf16(s[2 * j][0]), h01 = split_bf16(s[2 * j][1]);
          const float h10 = split_bf16(s[2 * j][2]), h11 = split_bf16(s[2 * j][3]);
          const float h20 = split_bf16(s[2 * j + 1][0]), h21 = split_bf16(s[2 * j + 1][1]);
          const float h30 = split_bf16(s[2 * j + 1][2]), h31 = split_bf16(s[2 * j + 1][3]);
          pa[part][j][0] = pack_bf16(h00, h01);
          pa[part][j][1] = pack_bf16(h10, h11);
          pa[part][j][2] = pack_bf16(h20, h21);
          pa[part][j][3] = pack_bf16(h30, h31);
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
                mma_bf16(o[2 * (v0 + vv)], pa[part][j], b[vv][0], b[vv][1]);
                mma_bf16(o[2 * (v0 + vv) + 1], pa[part][j], b[vv][2], b[vv][3]);
              }
            }
          }
        }
      }
    }
    __syncthreads();   // every warp is done with this tile's values
    if (more) load_v(k0 + kPN);   // lands during the next tile's score product
    cp_async_commit();
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (a.sink) {   // the sink joins the denominator once, on the scale of the row's running maximum
    const float sk = a.sink[h];
    l0 += expf(sk - m0);
    l1 += expf(sk - m1);
  }
  const bool pair_store = a.ld_out % 2 == 0;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = half ? r1 : r0;
    if (r >= count) continue;
    const int64_t t = first + r;
    const float k = a.out_scale / (half ? l1 : l0);
    const float* gt = a.gate ? a.gate + t * a.ld_gate + (int64_t)h * DV + 2 * t4 : nullptr;
    T* dst = a.out + t * a.ld_out + (int64_t)h * DV + 2 * t4;
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i) {
      const float g0 = gt ? 1.f / (1.f + expf(-gt[i * 8])) : 1.f, g1 = gt ? 1.f / (1.f + expf(-gt[i * 8 + 1])) : 1.f;
      const float y0 = o[i][2 * half] * k * g0, y1 = o[i][2 * half + 1] * k * g1;
      if (pair_store) {
        *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(y0, y1);
      } else {   // rows of odd length: every other row starts on an odd element
        dst[i * 8] = __float2bfloat16_rn(y0);
        dst[i * 8 + 1] = __float2bfloat16_rn(y1);
      }
    }
  }
}

inline size_t prompt_smem(int d, int dv) {
  return ((size_t)kPM * (d + kPad) + (size_t)kPN * (d + kPad) + (size_t)kPN * (dv + kPad)) * 2;
}

inline bool prompt_ok(int dt, int H, int G, int d, int dv) {
  if (dt != AO_LM_BF16 || G <= 0 || H % G || d <= 0 || d % 16 || dv % 16 || dv < 16 || dv > 128) return false;
  return prompt_smem(d, dv) <= 200 * 1024;
}

template <int NV>
int launch_prompt(const PromptArgs& a, int n_tiles, cudaStream_t st) {
  const size_t smem = prompt_smem(a.d, 16 * NV);
  auto kern = chunk_attention_prompt_kernel<NV>;
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

extern "C" int ao_lm_chunk_attention_prompt_plan(int dt, int H, int G, int d, int dv, int* tile_rows) {
  LM_CHECK_ARG(tile_rows);
  *tile_rows = prompt_ok(dt, H, G, d, dv) ? kPM : 0;
  return AO_B200_OK;
}

extern "C" int ao_lm_sink_attention_prompt(const float* qn, const void* kn, const void* vn, const void* ring_k,
                                           const void* ring_v, int dt, const float* gate, int64_t ld_gate,
                                           const float* dist_bias, int n_dist, const float* sink, const int32_t* slot,
                                           const int32_t* pos, const int32_t* back, const int32_t* tile_first,
                                           const int32_t* tile_count, int n_tiles, int H, int G, int d, int dv, int chunk,
                                           float scale, float softcap, float out_scale, void* out, int64_t ld_out,
                                           void* stream) {
  LM_CHECK_ARG(qn && kn && vn && ring_k && ring_v && slot && pos && back && tile_first && tile_count && out);
  LM_CHECK_ARG(n_tiles > 0 && (!dist_bias || n_dist > 0) && chunk > 0 && H > 0 && H <= 65535);
  if (!prompt_ok(dt, H, G, d, dv)) return AO_B200_ERR_UNSUPPORTED;
  // 16-byte copies of queries, keys and values; the result is stored in pairs when its rows allow it
  LM_CHECK_ARG(reinterpret_cast<uintptr_t>(out) % 4 == 0 && reinterpret_cast<uintptr_t>(qn) % 16 == 0 &&
               reinterpret_cast<uintptr_t>(kn) % 16 == 0 && reinterpret_cast<uintptr_t>(vn) % 16 == 0 &&
               reinterpret_cast<uintptr_t>(ring_k) % 16 == 0 && reinterpret_cast<uintptr_t>(ring_v) % 16 == 0);
  using T = __nv_bfloat16;
  PromptArgs a{qn, static_cast<const T*>(kn), static_cast<const T*>(vn), static_cast<const T*>(ring_k),
               static_cast<const T*>(ring_v), gate, ld_gate, dist_bias, n_dist, sink, slot, pos, back, tile_first, tile_count,
               H, G, d, chunk, scale, softcap, out_scale, static_cast<T*>(out), ld_out};
  const cudaStream_t st = lm_stream(stream);
#define LM_CP(NV) \
  case NV:        \
    return launch_prompt<NV>(a, n_tiles, st);
  switch (dv / 16) { LM_CP(1) LM_CP(2) LM_CP(3) LM_CP(4) LM_CP(5) LM_CP(6) LM_CP(7) LM_CP(8) }
#undef LM_CP
  return AO_B200_ERR_UNSUPPORTED;
}

extern "C" int ao_lm_chunk_attention_prompt(const float* qn, const void* kn, const void* vn, const void* ring_k,
                                            const void* ring_v, int dt, const float* gate, int64_t ld_gate,
                                            const float* dist_bias, int n_dist, const int32_t* slot, const int32_t* pos,
                                            const int32_t* back, const int32_t* tile_first, const int32_t* tile_count,
                                            int n_tiles, int H, int G, int d, int dv, int chunk, float scale, float softcap,
                                            float out_scale, void* out, int64_t ld_out, void* stream) {
  LM_CHECK_ARG(gate && dist_bias);
  return ao_lm_sink_attention_prompt(qn, kn, vn, ring_k, ring_v, dt, gate, ld_gate, dist_bias, n_dist, nullptr, slot, pos, back,
                                     tile_first, tile_count, n_tiles, H, G, d, dv, chunk, scale, softcap, out_scale, out, ld_out,
                                     stream);
}
