// q / k / v between the projections and the cache, in one pass (sm_100a).
//
//   v'  = lerp(v, v1, v_lamb)                                  torch.lerp, src/model/attn.py:105-107
//   q'  = rope(rms_norm(q)),  k' = rope(rms_norm(k))           src/model/attn.py:109-110
//
// A warp takes eight head rows of one token (batch row, token): the three positions and the lane's 16 bytes of
// the cos and sin rows are fetched once per warp, every row is read and written with 16-byte accesses (Dh / 8
// lanes per row, two or four rows per pass), and all loads of the warp are in flight before the first is used.
// A lane holds four of the pairs (x[2j], x[2j+1]) RoPE rotates.  The RMS over the row is a shuffle reduction in
// fp32 among the lanes of the row; the normalised row is rounded to the tensor dtype before the rotation, as the
// reference materialises it; products and sums of the rotation are rounded separately (no fused multiply-add),
// as eager PyTorch does.  HBM-bound byte work: every element is read once and written once.  Rows that are only
// 8-byte (Dh = 128) or 4-byte (Dh = 64) aligned take the older one-row-per-warp kernel below.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace we {

struct PrologueParams {
  const uint32_t* in[3];     // q, k, v rows as packed pairs
  const uint32_t* v1;
  uint16_t* out[3];
  int64_t in_s[3][3], v1_s[3], out_s[3][3];   // (b, h, t) strides in elements
  const void* v_lamb;
  int32_t v_lamb_dtype;
  const float* cos_t;
  const float* sin_t;
  int64_t table_rows;
  const int64_t* pos[3];     // t, y, x
  int64_t pos_bs;
  int32_t height, width;
  int32_t B, T, Hq, Hkv, Dh;
  int32_t bf16;
  float eps;
  int32_t* status;
};

constexpr int kPrologueThreads = 256;

template <bool BF16>
__device__ __forceinline__ float2 unpack_pair(uint32_t v) {
  if constexpr (BF16) {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xFFFF0000u));
  } else {
    return __half22float2(*reinterpret_cast<const __half2*>(&v));
  }
}
template <bool BF16>
__device__ __forceinline__ float round16(float x) {
  if constexpr (BF16) {
    return __bfloat162float(__float2bfloat16_rn(x));
  } else {
    return __half2float(__float2half_rn(x));
  }
}
template <bool BF16>
__device__ __forceinline__ uint16_t to16(float x) {
  if constexpr (BF16) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(x));
  } else {
    return __half_as_ushort(__float2half_rn(x));
  }
}

constexpr int kRowsPerWarp = 1;    // rows per warp (measured at the layer shape: 1 -> 5.4 us, 2 -> 6.0 us, 4 -> 7.8 us: more warps hide more latency)

template <bool BF16>
__global__ void __launch_bounds__(kPrologueThreads) qkv_prologue_kernel(const PrologueParams p) {
  // Programmatic dependent launch, both ways (as in the append kernel): wait for the kernel ahead, then let the
  // kernel behind (the attention of this layer-step) begin its on-chip set-up.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int slots = p.Hq + 2 * p.Hkv;                                   // q heads, k heads, v heads
  // (row indices fit 32 bits: the host rejects larger problems; 64-bit divisions would dominate the kernel)
  const uint32_t rows = static_cast<uint32_t>(p.B) * static_cast<uint32_t>(p.T) * static_cast<uint32_t>(slots);
  const uint32_t r0 = (blockIdx.x * (kPrologueThreads / 32) + (threadIdx.x >> 5)) * kRowsPerWarp;
  if (r0 >= rows) return;
  const int npair = p.Dh >> 6;                                          // pairs per lane: 1 (Dh=64) or 2 (Dh=128)
  const int half = p.Dh >> 1;
  // pair index of this lane's u-th pair
  auto pair_of = [&](int u) { return npair == 2 ? 2 * lane + u : lane; };
  auto load_row = [&](const uint32_t* src) {
    uint2 w = make_uint2(0u, 0u);
    if (npair == 2) w = reinterpret_cast<const uint2*>(src)[lane];      // rows are 8-byte aligned when Dh = 128
    else w.x = src[lane];
    return w;
  };

  // ---- phase 1: every load that depends on nothing but the row index
  int which[kRowsPerWarp];
  uint16_t* dst[kRowsPerWarp];
  uint2 raw[kRowsPerWarp], raw1[kRowsPerWarp];
  int64_t pt[kRowsPerWarp], py[kRowsPerWarp], px[kRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    const uint32_t r = r0 + i;
    which[i] = -1;
    if (r < rows) {
      const uint32_t bt = r / static_cast<uint32_t>(slots);
      const int slot = static_cast<int>(r - bt * slots);
      const int b = static_cast<int>(bt / static_cast<uint32_t>(p.T));
      const int t = static_cast<int>(bt - b * p.T);
      const int w = slot < p.Hq ? 0 : (slot < p.Hq + p.Hkv ? 1 : 2);
      const int h = w == 0 ? slot : (w == 1 ? slot - p.Hq : slot - p.Hq - p.Hkv);
      which[i] = w;
      dst[i] = p.out[w] + b * p.out_s[w][0] + h * p.out_s[w][1] + t * p.out_s[w][2];
      raw[i] = load_row(p.in[w] + ((b * p.in_s[w][0] + h * p.in_s[w][1] + t * p.in_s[w][2]) >> 1));
      raw1[i] = make_uint2(0u, 0u);
      pt[i] = py[i] = px[i] = 0;
      if (w == 2) {
        if (p.v1 != nullptr) raw1[i] = load_row(p.v1 + ((b * p.v1_s[0] + h * p.v1_s[1] + t * p.v1_s[2]) >> 1));
      } else {
        const int64_t pb = static_cast<int64_t>(b) * p.pos_bs + t;
        pt[i] = p.pos[0][pb];
        py[i] = p.pos[1][pb];
        px[i] = p.pos[2][pb];
      }
    }
  }
  float lamb = 0.f;
  if (p.v1 != nullptr) {
    if (p.v_lamb_dtype == WE_B200_F32) lamb = *static_cast<const float*>(p.v_lamb);
    else if (p.v_lamb_dtype == WE_B200_BF16) lamb = __bfloat162float(*static_cast<const __nv_bfloat16*>(p.v_lamb));
    else lamb = __half2float(*static_cast<const __half*>(p.v_lamb));
  }

  // ---- phase 2: the angle rows (RoPE.get_angles, src/model/attn.py:22-31), which need the positions
  float2 cs[kRowsPerWarp], sn[kRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    cs[i] = sn[i] = make_float2(0.f, 0.f);
    if (which[i] == 0 || which[i] == 1) {
      int64_t idx = pt[i] * (static_cast<int64_t>(p.height) * p.width) + py[i] * p.width + px[i];
      if (idx < 0 || idx >= p.table_rows) {
        if (lane == 0 && p.status != nullptr) atomicExch(p.status, WE_B200_ST_INDEX_RANGE);
        idx = idx < 0 ? 0 : p.table_rows - 1;
      }
      const float* ct = p.cos_t + idx * half;
      const float* st = p.sin_t + idx * half;
      if (npair == 2) {
        cs[i] = reinterpret_cast<const float2*>(ct)[lane];
        sn[i] = reinterpret_cast<const float2*>(st)[lane];
      } else {
        cs[i].x = ct[lane];
        sn[i].x = st[lane];
      }
    }
  }

  // ---- phase 3: arithmetic and stores
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    if (which[i] < 0) continue;                                          // (uniform over the warp)
    float2 x[2] = {unpack_pair<BF16>(raw[i].x), unpack_pair<BF16>(raw[i].y)};
    if (which[i] == 2) {
      // value residual: torch.lerp's two-sided form in fp32 (src/model/attn.py:105-107)
      if (p.v1 != nullptr) {
        const float2 e[2] = {unpack_pair<BF16>(raw1[i].x), unpack_pair<BF16>(raw1[i].y)};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const float d0 = __fsub_rn(e[u].x, x[u].x), d1 = __fsub_rn(e[u].y, x[u].y);
          if (fabsf(lamb) < 0.5f) {
            x[u].x = __fadd_rn(x[u].x, __fmul_rn(lamb, d0));
            x[u].y = __fadd_rn(x[u].y, __fmul_rn(lamb, d1));
          } else {
            const float om = __fsub_rn(1.0f, lamb);
            x[u].x = __fsub_rn(e[u].x, __fmul_rn(d0, om));
            x[u].y = __fsub_rn(e[u].y, __fmul_rn(d1, om));
          }
        }
      }
      const uint32_t a0 = static_cast<uint32_t>(to16<BF16>(x[0].x)) | (static_cast<uint32_t>(to16<BF16>(x[0].y)) << 16);
      const uint32_t a1 = static_cast<uint32_t>(to16<BF16>(x[1].x)) | (static_cast<uint32_t>(to16<BF16>(x[1].y)) << 16);
      if (npair == 2) reinterpret_cast<uint2*>(dst[i])[lane] = make_uint2(a0, a1);
      else reinterpret_cast<uint32_t*>(dst[i])[lane] = a0;
      continue;
    }
    // weightless RMS norm in fp32 (src/model/nn.py:55-56), rounded to the tensor dtype
    float ss = x[0].x * x[0].x + x[0].y * x[0].y + x[1].x * x[1].x + x[1].y * x[1].y;   // (second pair is 0 at Dh=64)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rinv = 1.0f / sqrtf(ss / static_cast<float>(p.Dh) + p.eps);
    const float c[2] = {cs[i].x, cs[i].y}, s[2] = {sn[i].x, sn[i].y};
    uint16_t y0[2], y1[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const float x0 = round16<BF16>(__fmul_rn(x[u].x, rinv)), x1 = round16<BF16>(__fmul_rn(x[u].y, rinv));
      y0[u] = to16<BF16>(__fsub_rn(__fmul_rn(x0, c[u]), __fmul_rn(x1, s[u])));   // RoPE.forward, src/model/attn.py:37-39
      y1[u] = to16<BF16>(__fadd_rn(__fmul_rn(x1, c[u]), __fmul_rn(x0, s[u])));
    }
    if (npair == 2) {
      // first components of pairs 2 lane, 2 lane + 1 are neighbours in the first half; second components likewise
      reinterpret_cast<uint32_t*>(dst[i])[lane] = static_cast<uint32_t>(y0[0]) | (static_cast<uint32_t>(y0[1]) << 16);
      reinterpret_cast<uint32_t*>(dst[i] + half)[lane] = static_cast<uint32_t>(y1[0]) | (static_cast<uint32_t>(y1[1]) << 16);
    } else {
      dst[i][pair_of(0)] = y0[0];
      dst[i][half + pair_of(0)] = y1[0];
    }
  }
}


// ---------------------------------------------------------------- eight rows of one token per warp
#ifndef WE_PROLOGUE_ROWS_PER_WARP
#define WE_PROLOGUE_ROWS_PER_WARP 8
#endif
constexpr int kRowsPerGroup = WE_PROLOGUE_ROWS_PER_WARP;
// Threads per CTA of this kernel.  Small CTAs spread the warps evenly: the layer shape has 1536 warps for 148 SMs,
// which CTAs of eight warps deal out as one or two CTAs per SM (8 or 16 warps), CTAs of four as two or three.
#ifndef WE_PROLOGUE_TOKEN_THREADS
#define WE_PROLOGUE_TOKEN_THREADS 128
#endif
constexpr int kTokenThreads = WE_PROLOGUE_TOKEN_THREADS;

// two floats -> two 16-bit values in one word (first argument in the low half), round to nearest even
template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if constexpr (BF16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  } else {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}

template <bool BF16, int DH>
__global__ void __launch_bounds__(kTokenThreads) qkv_prologue_token_kernel(const PrologueParams p) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int kLanesPerRow = DH / 8;                  // 16 bytes per lane
  constexpr int kRowsPerPass = 32 / kLanesPerRow;       // 2 (Dh = 128) or 4 (Dh = 64)
  constexpr int kPasses = kRowsPerGroup / kRowsPerPass;
  constexpr int kHalf = DH / 2;
  const int lane = threadIdx.x & 31;
  const int hl = lane % kLanesPerRow;                    // lane within the row: elements [8 hl, 8 hl + 8)
  const int hr = lane / kLanesPerRow;                    // which row of the pass
  const int slots = p.Hq + 2 * p.Hkv;                    // q heads, k heads, v heads of a token
  const uint32_t groups = static_cast<uint32_t>((slots + kRowsPerGroup - 1) / kRowsPerGroup);
  const uint32_t wid = blockIdx.x * (kTokenThreads / 32) + (threadIdx.x >> 5);
  const uint32_t token = wid / groups;
  if (token >= static_cast<uint32_t>(p.B) * static_cast<uint32_t>(p.T)) return;
  const int grp = static_cast<int>(wid - token * groups);
  const int b = static_cast<int>(token / static_cast<uint32_t>(p.T));
  const int t = static_cast<int>(token - static_cast<uint32_t>(b) * p.T);

  // The positions head the longest chain of dependent loads (positions -> table row): they go out first.
  // (v rows are not rotated: a warp whose rows are all v rows skips the tables)
  const bool rotates = grp * kRowsPerGroup < p.Hq + p.Hkv;
  int64_t pos_t = 0, pos_y = 0, pos_x = 0;
  if (rotates) {
    const int64_t pb = static_cast<int64_t>(b) * p.pos_bs + t;
    pos_t = p.pos[0][pb];
    pos_y = p.pos[1][pb];
    pos_x = p.pos[2][pb];
  }
  // offsets of the token within each tensor, once per warp (the head's share is added per row)
  int64_t in_base[3], out_base[3];
#pragma unroll
  for (int w = 0; w < 3; ++w) {
    in_base[w] = b * p.in_s[w][0] + t * p.in_s[w][2] + 8 * hl;
    out_base[w] = b * p.out_s[w][0] + t * p.out_s[w][2] + 8 * hl;
  }
  const int64_t v1_base = b * p.v1_s[0] + t * p.v1_s[2] + 8 * hl;

  // ---- every load that depends on nothing but the indices: the rows, the residual rows, the positions
  int kind[kPasses];
  uint16_t* dst[kPasses];
  uint4 raw[kPasses], raw1[kPasses];
#pragma unroll
  for (int i = 0; i < kPasses; ++i) {
    const int slot = grp * kRowsPerGroup + i * kRowsPerPass + hr;
    kind[i] = -1;
    raw[i] = raw1[i] = make_uint4(0u, 0u, 0u, 0u);
    dst[i] = nullptr;
    if (slot < slots) {
      const int w = slot < p.Hq ? 0 : (slot < p.Hq + p.Hkv ? 1 : 2);
      const int h = w == 0 ? slot : (w == 1 ? slot - p.Hq : slot - p.Hq - p.Hkv);
      kind[i] = w;
      // (selects, not indexing: an array indexed at run time would live in local memory)
      const int64_t ib = w == 0 ? in_base[0] : (w == 1 ? in_base[1] : in_base[2]);
      const int64_t ob = w == 0 ? out_base[0] : (w == 1 ? out_base[1] : out_base[2]);
      dst[i] = p.out[w] + ob + h * p.out_s[w][1];
      const uint16_t* src = reinterpret_cast<const uint16_t*>(p.in[w]) + ib + h * p.in_s[w][1];
      raw[i] = *reinterpret_cast<const uint4*>(src);
      if (w == 2 && p.v1 != nullptr) {
        const uint16_t* s1 = reinterpret_cast<const uint16_t*>(p.v1) + v1_base + h * p.v1_s[1];
        raw1[i] = *reinterpret_cast<const uint4*>(s1);
      }
    }
  }
  float4 cs = make_float4(0.f, 0.f, 0.f, 0.f), sn = cs;
  if (rotates) {
    // the angle row of the token (RoPE.get_angles, src/model/attn.py:22-31): once per warp
    int64_t idx = pos_t * (static_cast<int64_t>(p.height) * p.width) + pos_y * p.width + pos_x;
    if (idx < 0 || idx >= p.table_rows) {
      if (lane == 0 && p.status != nullptr) atomicExch(p.status, WE_B200_ST_INDEX_RANGE);
      idx = idx < 0 ? 0 : p.table_rows - 1;
    }
    cs = *reinterpret_cast<const float4*>(p.cos_t + idx * kHalf + 4 * hl);
    sn = *reinterpret_cast<const float4*>(p.sin_t + idx * kHalf + 4 * hl);
  }
  float lamb = 0.f;
  if (p.v1 != nullptr) {
    if (p.v_lamb_dtype == WE_B200_F32) lamb = *static_cast<const float*>(p.v_lamb);
    else if (p.v_lamb_dtype == WE_B200_BF16) lamb = __bfloat162float(*static_cast<const __nv_bfloat16*>(p.v_lamb));
    else lamb = __half2float(*static_cast<const __half*>(p.v_lamb));
  }
  const float c[4] = {cs.x, cs.y, cs.z, cs.w}, s[4] = {sn.x, sn.y, sn.z, sn.w};

  // ---- arithmetic and stores
#pragma unroll
  for (int i = 0; i < kPasses; ++i) {
    const uint32_t rw[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
    float2 x[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) x[u] = unpack_pair<BF16>(rw[u]);
    if (kind[i] == 2) {
      // value residual: torch.lerp's two-sided form in fp32 (src/model/attn.py:105-107)
      if (p.v1 != nullptr) {
        const uint32_t r1[4] = {raw1[i].x, raw1[i].y, raw1[i].z, raw1[i].w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float2 e = unpack_pair<BF16>(r1[u]);
          const float d0 = __fsub_rn(e.x, x[u].x), d1 = __fsub_rn(e.y, x[u].y);
          if (fabsf(lamb) < 0.5f) {
            x[u].x = __fadd_rn(x[u].x, __fmul_rn(lamb, d0));
            x[u].y = __fadd_rn(x[u].y, __fmul_rn(lamb, d1));
          } else {
            const float om = __fsub_rn(1.0f, lamb);
            x[u].x = __fsub_rn(e.x, __fmul_rn(d0, om));
            x[u].y = __fsub_rn(e.y, __fmul_rn(d1, om));
          }
        }
      }
      uint4 o;
      o.x = pack16<BF16>(x[0].x, x[0].y);
      o.y = pack16<BF16>(x[1].x, x[1].y);
      o.z = pack16<BF16>(x[2].x, x[2].y);
      o.w = pack16<BF16>(x[3].x, x[3].y);
      *reinterpret_cast<uint4*>(dst[i]) = o;
    }
    // weightless RMS norm in fp32 (src/model/nn.py:55-56), rounded to the tensor dtype.  (Every lane takes part
    // in the shuffles; rows of other kinds and empty rows contribute to sums nobody reads.)
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u) ss += x[u].x * x[u].x + x[u].y * x[u].y;
#pragma unroll
    for (int o = kLanesPerRow / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (kind[i] == 0 || kind[i] == 1) {
      const float rinv = 1.0f / sqrtf(ss / static_cast<float>(DH) + p.eps);
      float y0[4], y1[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float x0 = round16<BF16>(__fmul_rn(x[u].x, rinv)), x1 = round16<BF16>(__fmul_rn(x[u].y, rinv));
        y0[u] = __fsub_rn(__fmul_rn(x0, c[u]), __fmul_rn(x1, s[u]));   // RoPE.forward, src/model/attn.py:37-39
        y1[u] = __fadd_rn(__fmul_rn(x1, c[u]), __fmul_rn(x0, s[u]));
      }
      // dst points at element 8 hl of the row; the lane's pairs are 4 hl .. 4 hl + 3: first components go to
      // elements [4 hl, 4 hl + 4) of the first half, second components to the same places of the second half
      uint16_t* row0 = dst[i] - 8 * hl;
      uint2 a, bb;
      a.x = pack16<BF16>(y0[0], y0[1]);
      a.y = pack16<BF16>(y0[2], y0[3]);
      bb.x = pack16<BF16>(y1[0], y1[1]);
      bb.y = pack16<BF16>(y1[2], y1[3]);
      *reinterpret_cast<uint2*>(row0 + 4 * hl) = a;
      *reinterpret_cast<uint2*>(row0 + kHalf + 4 * hl) = bb;
    }
  }
}

}  // namespace we

extern "C" int we_b200_qkv_prologue(const we_b200_prologue_args* a, int32_t* status, void* stream) {
  using namespace we;
  if (a == nullptr || !a->q_in || !a->k_in || !a->v_in || !a->q_out || !a->k_out || !a->v_out || !a->cos_table ||
      !a->sin_table || !a->t_pos || !a->y_pos || !a->x_pos)
    return WE_B200_E_NULL;
  if (a->v1 != nullptr && a->v_lamb == nullptr) return WE_B200_E_NULL;
  if (a->dtype != WE_B200_BF16 && a->dtype != WE_B200_F16) return WE_B200_E_DTYPE;
  if (a->Dh != 64 && a->Dh != 128) return WE_B200_E_DTYPE;
  if (a->v1 != nullptr && a->v_lamb_dtype != WE_B200_BF16 && a->v_lamb_dtype != WE_B200_F16 &&
      a->v_lamb_dtype != WE_B200_F32)
    return WE_B200_E_DTYPE;
  if (a->B < 1 || a->T < 1 || a->Hq < 1 || a->Hkv < 1 || a->height < 1 || a->width < 1 || a->table_rows < 1 ||
      a->pos_batch_stride < 0)
    return WE_B200_E_SHAPE;
  // rows are read as 8-byte (Dh = 128) or 4-byte (Dh = 64) words: strides and bases must be aligned to that
  const int64_t* strides[7] = {a->q_in_strides, a->k_in_strides, a->v_in_strides, a->v1_strides,
                               a->q_out_strides, a->k_out_strides, a->v_out_strides};
  for (int i = 0; i < 7; ++i) {
    if (i == 3 && a->v1 == nullptr) continue;
    for (int d = 0; d < 3; ++d) {
      if (strides[i][d] < 0) return WE_B200_E_SHAPE;
      if (strides[i][d] & (a->Dh == 128 ? 3 : 1)) return WE_B200_E_ALIGN;
    }
  }
  const void* ptrs[7] = {a->q_in, a->k_in, a->v_in, a->v1, a->q_out, a->k_out, a->v_out};
  for (int i = 0; i < 7; ++i)
    if (ptrs[i] != nullptr && (reinterpret_cast<uintptr_t>(ptrs[i]) & (a->Dh == 128 ? 7u : 3u))) return WE_B200_E_ALIGN;

  PrologueParams p;
  p.in[0] = static_cast<const uint32_t*>(a->q_in);
  p.in[1] = static_cast<const uint32_t*>(a->k_in);
  p.in[2] = static_cast<const uint32_t*>(a->v_in);
  p.v1 = static_cast<const uint32_t*>(a->v1);
  p.out[0] = static_cast<uint16_t*>(a->q_out);
  p.out[1] = static_cast<uint16_t*>(a->k_out);
  p.out[2] = static_cast<uint16_t*>(a->v_out);
  for (int d = 0; d < 3; ++d) {
    p.in_s[0][d] = a->q_in_strides[d];
    p.in_s[1][d] = a->k_in_strides[d];
    p.in_s[2][d] = a->v_in_strides[d];
    p.v1_s[d] = a->v1 != nullptr ? a->v1_strides[d] : 0;
    p.out_s[0][d] = a->q_out_strides[d];
    p.out_s[1][d] = a->k_out_strides[d];
    p.out_s[2][d] = a->v_out_strides[d];
  }
  p.v_lamb = a->v_lamb;
  p.v_lamb_dtype = a->v_lamb_dtype;
  p.cos_t = a->cos_table;
  p.sin_t = a->sin_table;
  p.table_rows = a->table_rows;
  p.pos[0] = a->t_pos;
  p.pos[1] = a->y_pos;
  p.pos[2] = a->x_pos;
  p.pos_bs = a->pos_batch_stride;
  p.height = a->height;
  p.width = a->width;
  p.B = a->B;
  p.T = a->T;
  p.Hq = a->Hq;
  p.Hkv = a->Hkv;
  p.Dh = a->Dh;
  p.bf16 = a->dtype == WE_B200_BF16;
  p.eps = a->eps;
  p.status = status;

  const int64_t rows = static_cast<int64_t>(a->B) * a->T * (a->Hq + 2 * a->Hkv);
  // 16-byte aligned rows (the merged-QKV slices are): eight rows of a token per warp; otherwise one row per warp
  bool wide = true;
  for (int i = 0; i < 7; ++i) {
    if (ptrs[i] == nullptr) continue;
    if (reinterpret_cast<uintptr_t>(ptrs[i]) & 15u) wide = false;
    for (int d = 0; d < 3; ++d)
      if (strides[i][d] & 7) wide = false;
  }
  if ((reinterpret_cast<uintptr_t>(a->cos_table) | reinterpret_cast<uintptr_t>(a->sin_table)) & 15u) wide = false;
  const int64_t groups = (a->Hq + 2 * a->Hkv + kRowsPerGroup - 1) / kRowsPerGroup;
  const int64_t per_block = wide ? (kTokenThreads / 32) : (kPrologueThreads / 32) * kRowsPerWarp;
  const int64_t units = wide ? static_cast<int64_t>(a->B) * a->T * groups : rows;
  const int64_t blocks = (units + per_block - 1) / per_block;
  if (blocks > 0x7FFFFFFF || rows > 0x7FFFFFFF || units > 0x7FFFFFFF) return WE_B200_E_LIMIT;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
  cfg.blockDim = dim3(wide ? kTokenThreads : kPrologueThreads, 1, 1);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  if (wide && p.Dh == 128) {
    e = p.bf16 ? cudaLaunchKernelEx(&cfg, qkv_prologue_token_kernel<true, 128>, p)
               : cudaLaunchKernelEx(&cfg, qkv_prologue_token_kernel<false, 128>, p);
  } else if (wide) {
    e = p.bf16 ? cudaLaunchKernelEx(&cfg, qkv_prologue_token_kernel<true, 64>, p)
               : cudaLaunchKernelEx(&cfg, qkv_prologue_token_kernel<false, 64>, p);
  } else {
    e = p.bf16 ? cudaLaunchKernelEx(&cfg, qkv_prologue_kernel<true>, p)
               : cudaLaunchKernelEx(&cfg, qkv_prologue_kernel<false>, p);
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (e != cudaSuccess) return static_cast<int>(e);
  const cudaError_t e2 = cudaGetLastError();
  return e2 == cudaSuccess ? WE_B200_OK : static_cast<int>(e2);
}
