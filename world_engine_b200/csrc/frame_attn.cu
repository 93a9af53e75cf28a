// Frame-causal attention over the KV ring-buffer cache (sm_100a).
//
// The T queries of the new frame attend to every visible token of the cache:
// all tokens with written != 0 except the ring slot the frame maps to on a
// write step, plus the tail frame (LayerKVCache.upsert's mask,
// src/model/kv_cache.py:141-144, fed to flex_attention at
// src/model/attn.py:116).  Keys are consumed where they lie: the physical
// buffer [0, L+T) is cut into 128-key tiles, each CTA builds the list of
// tiles that hold a visible key from `written` and the device-resident frame
// counter, and walks its share of that list.  Ring wrap-around therefore is
// only "which tiles are listed"; nothing is gathered or copied.
//
// One CTA = 128 queries of one (batch row, head) x one split of the tile
// list.  Warp roles (192 threads):
//   warps 0-3  softmax: thread r owns query row r (TMEM lane r); online
//              softmax in fp32 with exp2 and a lazily updated row maximum;
//              writes P (bf16/f16) back to tensor memory; rescales O only
//              when a row maximum grew by more than 2^8.
//   warp 4     producer: TMA loads of Q once and of K / V tiles through a
//              ring of shared-memory stages guarded by mbarriers.
//   warp 5     MMA issuer: tcgen05.mma S = Q K^T (both operands in shared
//              memory, K-major, 128-byte swizzle) into one of two S buffers in
//              tensor memory, and O += P V with P read from tensor memory
//              and V from shared memory (MN-major).  Owns the TMEM allocation.
// S is double-buffered so the tensor pipe computes S(i+1) while the softmax
// warps work on S(i).
//
// Split-KV: when (batch x heads x query tiles) cannot fill the SMs, the tile
// list is split over several CTAs.  Each writes its un-normalised O, row
// maxima and row sums to the workspace; the CTA that arrives last at a
// per-(row, head, query tile) ticket counter merges them in a fixed order and
// writes the output.  Nobody spins on another CTA.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace we {

constexpr int kBlockM = 128;    // queries per CTA (= TMEM lanes)
constexpr int kBlockN = 128;    // keys per tile
constexpr int kMaxTiles = 1024; // capacity limit: 131072 tokens per (row, head)
constexpr int kAttnThreads = 192;
constexpr int kMaxSplits = 32;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO = 256, kColP0 = 384, kColP1 = 448;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

template <int DH>
struct AttnCfg {
  static constexpr int kChunks = DH / 64;                 // 128-byte column chunks per row
  static constexpr int kChunkBytes = kBlockN * 128;       // one chunk of a 128-row tile
  static constexpr int kTileBytes = kChunks * kChunkBytes;
  static constexpr int kStages = DH == 128 ? 2 : 4;       // K/V stages; keeps smem > half an SM
  static constexpr int kSmemTiles = kTileBytes * (1 + 2 * kStages);
  static constexpr int kSmemAux = 64 * 8 + kMaxTiles * 4 + kMaxTiles * 2 + 64;
  static constexpr int kSmemBytes = kSmemTiles + kSmemAux + 1024;  // + slack for 1024-byte alignment
};

struct AttnParams {
  void* out;
  int64_t os[3];                 // out strides (b, h, t) in elements
  const uint8_t* written;
  const int64_t* frame_t;
  int64_t written_batch_stride;
  int64_t frame_t_stride;
  int64_t L;
  int32_t C;                     // L + T
  int32_t T, Hq, Hkv, dilation;
  int32_t ntiles;                // ceil(C / 128)
  int32_t nsplit, n_qtiles;
  int32_t q_perm[3];             // which of (t, h, b) feeds tensor-map coordinate 1, 2, 3
  int32_t kv_perm[3];
  float scale_log2;
  float* ws_o;                   // [unit][split][DH][128]
  float* ws_ml;                  // [unit][split][2][128]
  int32_t* ws_cnt;               // [unit]
  int32_t* status;
};

#ifdef WE_ATTN_DEBUG
// Debug builds only: descriptor fields overridable at run time (0 = keep the default), and a
// per-CTA timeline (SM cycles since the CTA started) written to a caller-provided buffer.
__constant__ uint32_t g_dbg[8];
__device__ uint32_t* g_trace = nullptr;
#define WE_TRACE(slot)                                                                             \
  do {                                                                                             \
    if (trace != nullptr) trace[(slot)] = static_cast<uint32_t>(clock64() - t_start);              \
  } while (0)
#define WE_TRACE_VAL(slot, val)                                                                    \
  do {                                                                                             \
    if (trace != nullptr) trace[(slot)] = static_cast<uint32_t>(val);                              \
  } while (0)
#else
#define WE_TRACE(slot) do {} while (0)
#define WE_TRACE_VAL(slot, val) do {} while (0)
#endif

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

template <int DH, bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 1)
frame_attn_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  using Cfg = AttnCfg<DH>;
  constexpr int kStages = Cfg::kStages;
  constexpr uint32_t kInFmt = BF16 ? 1u : 0u;
  constexpr uint32_t kIdescS = umma_idesc(kInFmt, 0u, kBlockM, kBlockN);
  constexpr uint32_t kIdescPV = umma_idesc(kInFmt, 1u, kBlockM, DH);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::kTileBytes;
  uint8_t* sV = sK + kStages * Cfg::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kStages * Cfg::kTileBytes);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;              // [kStages]
  uint64_t* v_full = bars + 1 + kStages;    // [kStages]
  uint64_t* kv_empty = bars + 1 + 2 * kStages;  // [kStages]
  uint64_t* s_ready = bars + 1 + 3 * kStages;   // [2]
  uint64_t* p_ready = s_ready + 2;              // [2]
  uint64_t* o_ready = p_ready + 2;              // [1]
  uint32_t* s_cnt = reinterpret_cast<uint32_t*>(bars + 64);       // [kMaxTiles] visible keys per tile
  uint16_t* s_list = reinterpret_cast<uint16_t*>(s_cnt + kMaxTiles);  // [kMaxTiles] (tile << 1) | partial
  uint32_t* s_misc = reinterpret_cast<uint32_t*>(s_list + kMaxTiles);
  uint32_t* s_tmem = s_misc + 0;
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_misc + 1);
  uint32_t* s_nlist = s_misc + 2;
  uint32_t* s_ticket = s_misc + 3;
  int64_t* s_slot = reinterpret_cast<int64_t*>(s_misc + 4);       // [0] base, [1] hide flag

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int qt = blockIdx.x % p.n_qtiles;
  const int split = blockIdx.x / p.n_qtiles;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int kvh = h / (p.Hq / p.Hkv);
  const int q0 = qt * kBlockM;
#ifdef WE_ATTN_DEBUG
  const long long t_start = clock64();
  uint32_t* trace = nullptr;
  {
    const unsigned cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    if (g_trace != nullptr && cta < 64u) trace = g_trace + cta * 256u;
    if (trace != nullptr && tid == 0) {
      uint32_t smid;
      asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
      trace[0] = static_cast<uint32_t>(global_timer_ns());
      trace[230] = smid;
    }
  }
#endif

  // ---------------------------------------------------------------- set-up
  if (tid == 0) *s_abort = 0;
  if (warp == 4 && lane == 0) {
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(&s_ready[0], 1);
    mbar_init(&s_ready[1], 1);
    mbar_init(&p_ready[0], 128);
    mbar_init(&p_ready[1], 128);
    mbar_init(o_ready, 1);
    fence_mbar_init();
    fence_proxy_async_smem();
    // Q tile: rows q0 .. q0+127 of (b, h); rows past T are zero-filled by TMA.
    mbar_arrive_expect_tx(q_full, Cfg::kTileBytes);
    const int v3[3] = {q0, h, b};
    for (int ch = 0; ch < Cfg::kChunks; ++ch)
      tma_load_4d(sQ + ch * Cfg::kChunkBytes, &tm_q, q_full, ch * 64, v3[p.q_perm[0]], v3[p.q_perm[1]],
                  v3[p.q_perm[2]]);
  }
  if (warp == 5) {
    tmem_alloc(s_tmem, kTmemCols);
    tmem_relinquish();
  }
  if (tid == 32) {
    const int64_t t = p.frame_t[static_cast<int64_t>(b) * p.frame_t_stride];
    const SlotInfo s = slot_of(t, p.L, p.T, p.dilation);
    s_slot[0] = s.base;
    s_slot[1] = s.write_step;
  }
  for (int j = tid; j < p.ntiles; j += kAttnThreads) s_cnt[j] = 0;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tid == 0) WE_TRACE(1);
  const uint32_t tmem_base = *s_tmem;
  const int64_t slot_base = s_slot[0];
  const bool hide = s_slot[1] != 0;
  const uint8_t* wr = p.written + static_cast<int64_t>(b) * p.written_batch_stride;

  // ------------------------------------------------ visible-tile list (per CTA)
  // Each thread inspects 16 tokens at a time and adds its visible count to the tile's counter.
  {
    const int nvec = (p.C + 15) >> 4;
    for (int v = tid; v < nvec; v += kAttnThreads) {
      const int k0 = v << 4;
      int cnt = 0;
      if (k0 + 16 <= p.C) {
        const uint4 w = *reinterpret_cast<const uint4*>(wr + k0);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int key = k0 + j;
          const bool in_slot = hide && key >= slot_base && key < slot_base + p.T;
          cnt += (((ww[j >> 2] >> ((j & 3) * 8)) & 0xFFu) != 0u && !in_slot) ? 1 : 0;
        }
      } else {
        for (int key = k0; key < p.C; ++key) {
          const bool in_slot = hide && key >= slot_base && key < slot_base + p.T;
          cnt += (wr[key] != 0 && !in_slot) ? 1 : 0;
        }
      }
      if (cnt) atomicAdd(&s_cnt[k0 >> 7], static_cast<uint32_t>(cnt));
    }
  }
  __syncthreads();
  if (warp == 0) {
    int n = 0;
    for (int base = 0; base < p.ntiles; base += 32) {
      const int j = base + lane;
      const uint32_t c = j < p.ntiles ? s_cnt[j] : 0u;
      const unsigned m = __ballot_sync(0xffffffffu, c != 0u);
      if (c != 0u) s_list[n + __popc(m & ((1u << lane) - 1u))] = static_cast<uint16_t>((j << 1) | (c != kBlockN ? 1 : 0));
      n += __popc(m);
    }
    if (lane == 0) *s_nlist = n;
  }
  __syncthreads();
  const int n_list = static_cast<int>(*s_nlist);
  const int t0 = static_cast<int>((static_cast<int64_t>(n_list) * split) / p.nsplit);
  const int t1 = static_cast<int>((static_cast<int64_t>(n_list) * (split + 1)) / p.nsplit);
  const int n = t1 - t0;
  if (tid == 0) { WE_TRACE(2); WE_TRACE_VAL(3, n); }

  // ------------------------------------------------------------------ roles
  if (warp == 4) {
    if (lane == 0) {
      for (int i = 0; i < n; ++i) {
        const int st = i % kStages;
        if (i >= kStages) mbar_wait(&kv_empty[st], ((i / kStages) - 1) & 1, s_abort);
        if (i < 32) WE_TRACE(192 + i);
        const int key0 = (s_list[t0 + i] >> 1) * kBlockN;
        const int v3[3] = {key0, kvh, b};
        const int c1 = v3[p.kv_perm[0]], c2 = v3[p.kv_perm[1]], c3 = v3[p.kv_perm[2]];
        mbar_arrive_expect_tx(&k_full[st], Cfg::kTileBytes);
        for (int ch = 0; ch < Cfg::kChunks; ++ch)
          tma_load_4d(sK + st * Cfg::kTileBytes + ch * Cfg::kChunkBytes, &tm_k, &k_full[st], ch * 64, c1, c2, c3);
        mbar_arrive_expect_tx(&v_full[st], Cfg::kTileBytes);
        for (int ch = 0; ch < Cfg::kChunks; ++ch)
          tma_load_4d(sV + st * Cfg::kTileBytes + ch * Cfg::kChunkBytes, &tm_v, &v_full[st], ch * 64, c1, c2, c3);
      }
      if (n == 0) mbar_wait(q_full, 0, s_abort);  // nobody else consumes Q: let the copy land before exit
    }
  } else if (warp == 5) {
    if (lane == 0 && n > 0) {
      const uint32_t q_addr = smem_u32(sQ);
      const uint32_t k_addr = smem_u32(sK);
      const uint32_t v_addr = smem_u32(sV);
      mbar_wait(q_full, 0, s_abort);
      // S(i) = Q K(i)^T : M=128 queries, N=128 keys, K=DH in steps of 16.
      auto issue_s = [&](int i) {
        const int st = i % kStages;
        mbar_wait(&k_full[st], (i / kStages) & 1, s_abort);
        tc_fence_after();
        const uint32_t d = tmem_base + ((i & 1) ? kColS1 : kColS0);
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint32_t off = (kk >> 2) * Cfg::kChunkBytes + (kk & 3) * 32;
          const uint64_t a = umma_desc_sw128(q_addr + off, 16, 1024);
          const uint64_t bd = umma_desc_sw128(k_addr + st * Cfg::kTileBytes + off, 16, 1024);
          umma_ss(d, a, bd, kIdescS, kk > 0 ? 1u : 0u);
        }
        tc_commit(&s_ready[i & 1]);
      };
      issue_s(0);
      for (int i = 0; i < n; ++i) {
        const int st = i % kStages;
        if (i + 1 < n) issue_s(i + 1);
        mbar_wait(&p_ready[i & 1], (i >> 1) & 1, s_abort);
        if (i < 24) WE_TRACE(144 + 2 * i);
        mbar_wait(&v_full[st], (i / kStages) & 1, s_abort);
        if (i < 24) WE_TRACE(145 + 2 * i);
        tc_fence_after();
        // O += P(i) V(i) : M=128 queries, N=DH, K=128 keys in steps of 16.
        const uint32_t d = tmem_base + kColO;
        const uint32_t a_t = tmem_base + ((i & 1) ? kColP1 : kColP0);
        uint32_t v_lbo = Cfg::kChunkBytes, v_sbo = 1024, v_kstep = 2048, idesc_pv = kIdescPV;
#ifdef WE_ATTN_DEBUG
        if (g_dbg[0]) v_lbo = g_dbg[0];
        if (g_dbg[1]) v_sbo = g_dbg[1];
        if (g_dbg[2]) v_kstep = g_dbg[2];
        if (g_dbg[3]) idesc_pv = g_dbg[3];
#endif
#pragma unroll
        for (int kk = 0; kk < kBlockN / 16; ++kk) {
          const uint64_t bd = umma_desc_sw128(v_addr + st * Cfg::kTileBytes + kk * v_kstep, v_lbo, v_sbo);
          umma_ts(d, a_t + kk * 8, bd, idesc_pv, (i > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&kv_empty[st]);
        tc_commit(o_ready);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------- softmax warps
    const int row = tid;  // query row within the tile == TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    float m_run = -INFINITY;  // running row maximum, log2 domain, possibly stale by <= threshold
    float l_run = 0.f;
    for (int i = 0; i < n; ++i) {
      const int buf = i & 1;
      const uint32_t s_addr = tmem_base + lane_base + (buf ? kColS1 : kColS0);
      const uint32_t p_addr = tmem_base + lane_base + (buf ? kColP1 : kColP0);
      mbar_wait(&s_ready[buf], (i >> 1) & 1, s_abort);
      if (tid == 0 && i < 32) WE_TRACE(16 + 4 * i);
      tc_fence_after();
      uint32_t s[4][32];
      tmem_ld32(s_addr + 0, s[0]);
      tmem_ld32(s_addr + 32, s[1]);
      tmem_ld32(s_addr + 64, s[2]);
      tmem_ld32(s_addr + 96, s[3]);
      tmem_ld_wait();
      const uint32_t entry = s_list[t0 + i];
      if (entry & 1u) {
        // partial tile: mask tokens that are unwritten, hidden, or beyond the buffer
        const int key0 = static_cast<int>(entry >> 1) * kBlockN;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int key = key0 + c * 32 + j;
            bool vis = key < p.C;
            if (vis) vis = wr[key] != 0 && !(hide && key >= slot_base && key < slot_base + p.T);
            if (!vis) s[c][j] = 0xFF800000u;  // -inf
          }
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int j = 0; j < 32; ++j) mx = fmaxf(mx, __uint_as_float(s[c][j]));
      const float m_new = fmaxf(m_run, mx * p.scale_log2);
      if (tid == 0 && i < 32) WE_TRACE(17 + 4 * i);
      if (i > 0) {
        mbar_wait(o_ready, (i - 1) & 1, s_abort);  // O holds tiles < i and no MMA is writing it
        tc_fence_after();
      }
      if (tid == 0 && i < 32) WE_TRACE(18 + 4 * i);
      const bool need = (m_new - m_run) > kRescaleThreshold;  // first tile: inf > threshold
      if (__any_sync(0xffffffffu, need)) {
        const float alpha = exp2f(m_run - m_new);             // first tile: exp2(-inf) = 0
        l_run *= alpha;
        m_run = m_new;
        if (i > 0) {
#pragma unroll
          for (int c = 0; c < DH / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tmem_base + lane_base + kColO + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
            tmem_st32(tmem_base + lane_base + kColO + c * 32, o);
          }
        }
      }
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float p0 = exp2f(fmaf(__uint_as_float(s[c][2 * j]), p.scale_log2, -m_run));
          const float p1 = exp2f(fmaf(__uint_as_float(s[c][2 * j + 1]), p.scale_log2, -m_run));
          sum += p0 + p1;
          pk[j] = pack2<BF16>(p0, p1);
        }
        tmem_st16(p_addr + c * 16, pk);
      }
      l_run += sum;
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_ready[buf]);
      if (tid == 0 && i < 32) WE_TRACE(19 + 4 * i);
    }

    // ------------------------------------------------------------ epilogue
    if (n > 0) {
      mbar_wait(o_ready, (n - 1) & 1, s_abort);
      tc_fence_after();
    }
    if (tid == 0) WE_TRACE(224);
    const int unit = (b * p.Hq + h) * p.n_qtiles + qt;
    if (p.nsplit == 1) {
      const float inv = 1.0f / l_run;
      const bool in_range = q0 + row < p.T;
      uint8_t* orow = static_cast<uint8_t*>(p.out) +
                      2 * (b * p.os[0] + h * p.os[1] + static_cast<int64_t>(q0 + row) * p.os[2]);
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_base + lane_base + kColO + c * 32, o);
        tmem_ld_wait();
        if (in_range) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = pack2<BF16>(__uint_as_float(o[8 * j + 0]) * inv, __uint_as_float(o[8 * j + 1]) * inv);
            v.y = pack2<BF16>(__uint_as_float(o[8 * j + 2]) * inv, __uint_as_float(o[8 * j + 3]) * inv);
            v.z = pack2<BF16>(__uint_as_float(o[8 * j + 4]) * inv, __uint_as_float(o[8 * j + 5]) * inv);
            v.w = pack2<BF16>(__uint_as_float(o[8 * j + 6]) * inv, __uint_as_float(o[8 * j + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 64 + j * 16) = v;
          }
        }
      }
    } else {
      // Partial result of this split, column-major so that the 128 row-threads store coalesced.
      float* wo = p.ws_o + (static_cast<int64_t>(unit) * p.nsplit + split) * (DH * kBlockM);
      float* wml = p.ws_ml + (static_cast<int64_t>(unit) * p.nsplit + split) * (2 * kBlockM);
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t o[32];
        if (n > 0) {
          tmem_ld32(tmem_base + lane_base + kColO + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) __stcg(wo + (c * 32 + j) * kBlockM + row, __uint_as_float(o[j]));
      }
      __stcg(wml + row, m_run);
      __stcg(wml + kBlockM + row, l_run);
      __threadfence();
      named_bar_sync(1, 128);
      if (tid == 0) WE_TRACE(225);
      if (tid == 0) *s_ticket = static_cast<uint32_t>(atomicAdd(p.ws_cnt + unit, 1));
      named_bar_sync(1, 128);
      if (tid == 0) { WE_TRACE(226); WE_TRACE_VAL(229, *s_ticket); }
      if (*s_ticket == static_cast<uint32_t>(p.nsplit - 1)) {
        // Last split to arrive merges all of them, always in split order (deterministic).
        __threadfence();
        const float* ml0 = p.ws_ml + static_cast<int64_t>(unit) * p.nsplit * (2 * kBlockM);
        const float* o0 = p.ws_o + static_cast<int64_t>(unit) * p.nsplit * (DH * kBlockM);
        float m_all = -INFINITY;
        for (int s2 = 0; s2 < p.nsplit; ++s2) {
          const float ls = __ldcg(ml0 + s2 * 2 * kBlockM + kBlockM + row);
          const float ms = __ldcg(ml0 + s2 * 2 * kBlockM + row);
          if (ls > 0.f) m_all = fmaxf(m_all, ms);
        }
        float acc[DH];
#pragma unroll
        for (int j = 0; j < DH; ++j) acc[j] = 0.f;
        float den = 0.f;
        for (int s2 = 0; s2 < p.nsplit; ++s2) {
          const float ls = __ldcg(ml0 + s2 * 2 * kBlockM + kBlockM + row);
          const float ms = __ldcg(ml0 + s2 * 2 * kBlockM + row);
          if (!(ls > 0.f)) continue;
          const float wgt = exp2f(ms - m_all);
          den += ls * wgt;
          const float* os2 = o0 + static_cast<int64_t>(s2) * (DH * kBlockM) + row;
#pragma unroll
          for (int j = 0; j < DH; ++j) acc[j] = fmaf(wgt, __ldcg(os2 + j * kBlockM), acc[j]);
        }
        const float inv = 1.0f / den;
        if (q0 + row < p.T) {
          uint8_t* orow = static_cast<uint8_t*>(p.out) +
                          2 * (b * p.os[0] + h * p.os[1] + static_cast<int64_t>(q0 + row) * p.os[2]);
#pragma unroll
          for (int j = 0; j < DH / 8; ++j) {
            uint4 v;
            v.x = pack2<BF16>(acc[8 * j + 0] * inv, acc[8 * j + 1] * inv);
            v.y = pack2<BF16>(acc[8 * j + 2] * inv, acc[8 * j + 3] * inv);
            v.z = pack2<BF16>(acc[8 * j + 4] * inv, acc[8 * j + 5] * inv);
            v.w = pack2<BF16>(acc[8 * j + 6] * inv, acc[8 * j + 7] * inv);
            *reinterpret_cast<uint4*>(orow + j * 16) = v;
          }
        }
        if (tid == 0) p.ws_cnt[unit] = 0;  // leave the counter ready for the next launch
        if (tid == 0) WE_TRACE(227);
      }
    }
  }

  // --------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (tid == 0) WE_TRACE(228);
  if (*s_abort != 0) {
    if (tid == 0 && p.status != nullptr) atomicExch(p.status, WE_B200_ST_WAIT_EXPIRED);
    __nanosleep(1000000);  // let copies and MMAs that are still in flight land before the CTA goes away
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
    if (qres != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// Tensor map over a [B, H, N, Dh] view (Dh contiguous) with box (64, 128, 1, 1) and 128-byte swizzle.
// The three outer axes are ordered by stride as the encoder expects; perm[i] tells the kernel which of
// (n, h, b) feeds coordinate i+1.
static int make_map(CUtensorMap* m, const void* base, int dtype, int64_t N, int64_t H, int64_t B, int Dh,
                    const int64_t strides_bhn[3], int32_t perm[3]) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return WE_B200_E_DRIVER;
  struct Ax { int64_t size, stride; uint32_t box; int src; };
  Ax ax[3] = {{N, strides_bhn[2], 128u, 0}, {H, strides_bhn[1], 1u, 1}, {B, strides_bhn[0], 1u, 2}};
  // size-1 axes carry meaningless strides: park them at the end
  for (int i = 0; i < 3; ++i)
    for (int j = i + 1; j < 3; ++j) {
      const bool i_one = ax[i].size == 1, j_one = ax[j].size == 1;
      const bool swap = (i_one && !j_one) || (i_one == j_one && !i_one && ax[j].stride < ax[i].stride);
      if (swap) { Ax t = ax[i]; ax[i] = ax[j]; ax[j] = t; }
    }
  int64_t span = static_cast<int64_t>(Dh);
  for (int i = 0; i < 3; ++i) {
    if (ax[i].size == 1) ax[i].stride = span;  // any legal value
    if (ax[i].stride * 2 >= (1ll << 40)) return WE_B200_E_LIMIT;
    const int64_t reach = ax[i].stride * ax[i].size;
    if (reach > span) span = reach;
    if (ax[i].size > 0xFFFFFFFFll) return WE_B200_E_LIMIT;
  }
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(Dh), static_cast<cuuint64_t>(ax[0].size),
                              static_cast<cuuint64_t>(ax[1].size), static_cast<cuuint64_t>(ax[2].size)};
  const cuuint64_t gstr[3] = {static_cast<cuuint64_t>(ax[0].stride * 2), static_cast<cuuint64_t>(ax[1].stride * 2),
                              static_cast<cuuint64_t>(ax[2].stride * 2)};
  const cuuint32_t box[4] = {64u, ax[0].box, ax[1].box, ax[2].box};
  const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  for (int i = 0; i < 3; ++i) perm[i] = ax[i].src;
  const CUtensorMapDataType dt = dtype == WE_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = fn(m, dt, 4, const_cast<void*>(base), dims, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? WE_B200_OK : WE_B200_E_DRIVER;
}

static int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

struct SplitPlan {
  int n_qtiles, units, ntiles, nsplit;
  size_t o_bytes, ml_bytes, cnt_bytes;
};

static SplitPlan plan_splits(int B, int Hq, int T, int Dh, int64_t L) {
  SplitPlan s;
  s.n_qtiles = (T + kBlockM - 1) / kBlockM;
  s.units = B * Hq * s.n_qtiles;
  s.ntiles = static_cast<int>((L + T + kBlockN - 1) / kBlockN);
  const int sms = sm_count();
  int ns = s.units >= sms ? 1 : sms / s.units;
  if (ns > s.ntiles) ns = s.ntiles;
  if (ns > kMaxSplits) ns = kMaxSplits;
  if (ns < 1) ns = 1;
  s.nsplit = ns;
  s.o_bytes = ns > 1 ? static_cast<size_t>(s.units) * ns * Dh * kBlockM * sizeof(float) : 0;
  s.ml_bytes = ns > 1 ? static_cast<size_t>(s.units) * ns * 2 * kBlockM * sizeof(float) : 0;
  s.cnt_bytes = ((static_cast<size_t>(s.units) * sizeof(int32_t)) + 255) & ~static_cast<size_t>(255);
  return s;
}

template <int DH, bool BF16>
static int launch_variant(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p,
                          dim3 grid, cudaStream_t stream) {
  using Cfg = AttnCfg<DH>;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    const cudaError_t e = cudaFuncSetAttribute(frame_attn_kernel<DH, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               Cfg::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_done[dev] = true;
  }
  frame_attn_kernel<DH, BF16><<<grid, kAttnThreads, Cfg::kSmemBytes, stream>>>(tq, tk, tv, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? WE_B200_OK : static_cast<int>(e);
}

int frame_attn_launch(const void* q, const int64_t* qs, void* out, const int64_t* os, int Hq, const void* kv,
                      const uint8_t* written, const int64_t* frame_t, const we_b200_cache_geom* g, float scale,
                      void* workspace, size_t workspace_bytes, int32_t* status, cudaStream_t stream) {
  if (!q || !out || !kv || !written || !frame_t) return WE_B200_E_NULL;
  int rc = check_geom(g);
  if (rc != WE_B200_OK) return rc;
  if (g->dtype != WE_B200_BF16 && g->dtype != WE_B200_F16) return WE_B200_E_DTYPE;
  if (g->Dh != 64 && g->Dh != 128) return WE_B200_E_DTYPE;
  if (Hq < 1 || Hq % g->Hkv != 0) return WE_B200_E_SHAPE;
  if ((rc = check_strides(qs, 2)) != WE_B200_OK) return rc;
  if ((rc = check_strides(os, 2)) != WE_B200_OK) return rc;
  if (!aligned16(q) || !aligned16(out) || !aligned16(kv) || !aligned16(written)) return WE_B200_E_ALIGN;
  if (g->written_batch_stride % 16 != 0) return WE_B200_E_ALIGN;
  if ((g->written_batch_stride == 0) != (g->frame_t_stride == 0)) return WE_B200_E_SHAPE;
  const int64_t C = g->L + g->T;
  if (C > static_cast<int64_t>(kMaxTiles) * kBlockN) return WE_B200_E_LIMIT;
  if (g->B > 65535 || Hq > 65535) return WE_B200_E_LIMIT;

  const SplitPlan sp = plan_splits(g->B, Hq, g->T, g->Dh, g->L);
  const size_t need = sp.o_bytes + sp.ml_bytes + sp.cnt_bytes;
  if (sp.nsplit > 1) {
    if (workspace == nullptr || workspace_bytes < need) return WE_B200_E_WORKSPACE;
    if (!aligned16(workspace)) return WE_B200_E_ALIGN;
  }

  AttnParams p;
  p.out = out;
  for (int i = 0; i < 3; ++i) p.os[i] = os[i];
  p.written = written;
  p.frame_t = frame_t;
  p.written_batch_stride = g->written_batch_stride;
  p.frame_t_stride = g->frame_t_stride;
  p.L = g->L;
  p.C = static_cast<int32_t>(C);
  p.T = g->T;
  p.Hq = Hq;
  p.Hkv = g->Hkv;
  p.dilation = g->dilation;
  p.ntiles = sp.ntiles;
  p.nsplit = sp.nsplit;
  p.n_qtiles = sp.n_qtiles;
  p.scale_log2 = (scale > 0.f ? scale : 1.0f / sqrtf(static_cast<float>(g->Dh))) * 1.4426950408889634f;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  p.ws_cnt = reinterpret_cast<int32_t*>(ws);
  p.ws_ml = reinterpret_cast<float*>(ws + sp.cnt_bytes);
  p.ws_o = reinterpret_cast<float*>(ws + sp.cnt_bytes + sp.ml_bytes);
  p.status = status;
  CUtensorMap tq, tk, tv;
  const int64_t kvs[3] = {g->kv_batch_stride, C * g->Dh, static_cast<int64_t>(g->Dh)};
  if ((rc = make_map(&tq, q, g->dtype, g->T, Hq, g->B, g->Dh, qs, p.q_perm)) != WE_B200_OK) return rc;
  if ((rc = make_map(&tk, kv, g->dtype, C, g->Hkv, g->B, g->Dh, kvs, p.kv_perm)) != WE_B200_OK) return rc;
  int32_t perm_v[3];
  const uint8_t* v_base = static_cast<const uint8_t*>(kv) + 2 * g->kv_plane_stride;
  if ((rc = make_map(&tv, v_base, g->dtype, C, g->Hkv, g->B, g->Dh, kvs, perm_v)) != WE_B200_OK) return rc;

  dim3 grid(static_cast<unsigned>(sp.n_qtiles * sp.nsplit), static_cast<unsigned>(Hq), static_cast<unsigned>(g->B));
  if (g->Dh == 128) {
    return g->dtype == WE_B200_BF16 ? launch_variant<128, true>(tq, tk, tv, p, grid, stream)
                                    : launch_variant<128, false>(tq, tk, tv, p, grid, stream);
  }
  return g->dtype == WE_B200_BF16 ? launch_variant<64, true>(tq, tk, tv, p, grid, stream)
                                  : launch_variant<64, false>(tq, tk, tv, p, grid, stream);
}

}  // namespace we

#ifdef WE_ATTN_DEBUG
extern "C" __attribute__((visibility("default"))) int we_b200_debug_set(int idx, uint32_t value) {
  if (idx < 0 || idx >= 8) return -1;
  return static_cast<int>(cudaMemcpyToSymbol(we::g_dbg, &value, sizeof(value), idx * sizeof(uint32_t)));
}
// Buffer of 64 x 256 uint32 for the per-CTA timeline (null switches tracing off).
extern "C" __attribute__((visibility("default"))) int we_b200_debug_trace(uint32_t* buf) {
  return static_cast<int>(cudaMemcpyToSymbol(we::g_trace, &buf, sizeof(buf)));
}
#endif

extern "C" size_t we_b200_attn_workspace_bytes(int32_t B, int32_t Hq, int32_t T, int32_t Dh, int64_t L) {
  if (B < 1 || Hq < 1 || T < 1 || Dh < 1 || L < 1) return 0;
  const we::SplitPlan sp = we::plan_splits(B, Hq, T, Dh, L);
  return sp.o_bytes + sp.ml_bytes + sp.cnt_bytes;
}

extern "C" int we_b200_frame_attn(const void* q, const int64_t* q_strides_host, void* out,
                                  const int64_t* out_strides_host, int32_t Hq, const void* kv, const uint8_t* written,
                                  const int64_t* frame_t, const we_b200_cache_geom* geom_host, float scale,
                                  void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
  return we::frame_attn_launch(q, q_strides_host, out, out_strides_host, Hq, kv, written, frame_t, geom_host, scale,
                               workspace, workspace_bytes, status, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------- entry point that allocates nothing
// Some hosts of this library are not allowed to obtain device memory at all once they are running: a
// real-time frame loop that handed the whole GPU to its own arena at start-up and treats every later
// driver allocation as a fault (it may stall the device or fail when memory is fragmented), or a plug-in
// host that may only touch the buffers it is handed.  Such callers cannot provide the split-KV
// workspace.  For them the same attention kernel is offered with its scratch in a fixed array that is
// part of the loaded library image: every GPU that loads the library holds these bytes until the
// process exits, which is why the array is kept modest.
namespace we {
constexpr size_t kStaticScratchBytes = 12u << 20;  // 12 MiB: covers every split-KV plan on a 148-SM part at Dh <= 128
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
}  // namespace we

extern "C" int we_b200_frame_attn_static(const void* q, const int64_t* q_strides_host, void* out,
                                         const int64_t* out_strides_host, int32_t Hq, const void* kv,
                                         const uint8_t* written, const int64_t* frame_t,
                                         const we_b200_cache_geom* geom_host, float scale, int32_t* status,
                                         void* stream) {
  // In host code `g_static_scratch` is only a handle for the symbol, not a device address: the address
  // on the current device has to be asked for, once per device, with that device current.
  static std::mutex mu;
  static void* scratch_of_device[64] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return WE_B200_E_LIMIT;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (scratch_of_device[dev] == nullptr) {
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, we::g_static_scratch);
      if (e != cudaSuccess) return static_cast<int>(e);
      scratch_of_device[dev] = ptr;
    }
    scratch = scratch_of_device[dev];
  }
  if (geom_host == nullptr) return WE_B200_E_NULL;
  if (geom_host->B < 1 || Hq < 1 || geom_host->T < 1 || geom_host->Dh < 1 || geom_host->L < 1) return WE_B200_E_SHAPE;
  const we::SplitPlan sp = we::plan_splits(geom_host->B, Hq, geom_host->T, geom_host->Dh, geom_host->L);
  if (sp.o_bytes + sp.ml_bytes + sp.cnt_bytes > we::kStaticScratchBytes) return WE_B200_E_STATIC_SCRATCH;
  // The array keeps whatever the previous call left.  Only the arrival counters must start at zero (the
  // kernel restores them, but a call that was cut short may not have): clear them on the caller's stream.
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  e = cudaMemsetAsync(scratch, 0, sp.cnt_bytes, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  return we::frame_attn_launch(q, q_strides_host, out, out_strides_host, Hq, kv, written, frame_t, geom_host, scale,
                               scratch, we::kStaticScratchBytes, status, s);
}
