// Frame-causal attention over the KV ring-buffer cache (sm_100a).
//
// The T queries of the new frame attend to every visible token of the cache:
// all tokens with written != 0 except the ring slot the frame maps to on a
// write step, plus the tail frame (LayerKVCache.upsert's mask,
// src/model/kv_cache.py:141-144, fed to flex_attention at
// src/model/attn.py:116).  Keys are consumed where they lie: the physical
// buffer [0, L+T) is cut into 128-key tiles; tiles lying wholly in the hidden
// slot are excluded by arithmetic on the device-resident frame counter, the
// remaining candidates are divided among the CTAs that share a query tile, and
// each CTA scans `written` for its candidates and walks those that hold a
// visible key.  Ring wrap-around therefore is only "which tiles are walked";
// nothing is gathered or copied.
//
// One CTA = 128 queries of one (batch row, head) x one split of the key tiles.
// Warp roles (384 threads):
//   warps 0-3   softmax group 0, warps 4-7 softmax group 1.  Thread r of either
//               group owns query row r (TMEM lane r), so row max and row sum
//               are in-thread reductions.  Group g handles keys [64g, 64g+64)
//               of every tile as a stream of its own: running maximum, row
//               sum and accumulator O_g; the two streams are merged once at
//               the end.  exp2 with the scale folded in, arithmetic on packed
//               fp32 pairs; three pairs in four go through ex2.approx, the
//               fourth through a cubic on the FMA pipe (the special-function
//               unit is the busiest pipe of the loop); the running maximum
//               is raised (and O_g rescaled in tensor memory) only when it
//               grew by more than 2^8; P (bf16/f16) overwrites the S columns
//               the thread has consumed.
//   warp 8      producer: barrier set-up, Q load, the first two K/V tiles
//               (fetched before their visibility is known), then the K ring.
//               With the fused append, after the last tile of the walk it
//               does this CTA's share of persisting the new frame: it fetches
//               a new tile once more and writes it into the tail slice or the
//               ring slot with a tensor store from shared memory.
//   warp 10     V producer: the V tiles through a ring of their own.
//   warp 9      owns tensor memory; its first thread issues the tcgen05.mma
//               products of the even tiles: O_g += P_g V_g for both key halves
//               of tile i (P from tensor memory, V from shared memory as an
//               MN-major operand), then at once S(i+2) = Q K^T (both operands
//               in shared memory, K-major, 128-byte swizzle) into the S buffer
//               that P(i) occupied.
//   warp 11     compacts the visible-tile list, then its first thread issues
//               the products of the odd tiles the same way (issuing a product
//               blocks the thread about as long as the tensor pipe works on
//               it, so two threads keep the pipe fed); with the fused append,
//               marks the ring slot as written.
// Tensor memory (512 columns): S0, S1, O_0, O_1, 128 columns each.
// A completed S product frees its K stage and a completed P V product its V
// stage: one mbarrier each serves the softmax warps and the producer.
//
// The launch carries the programmatic-stream-serialization attribute: barrier
// set-up, tensor-memory allocation and tensor-map prefetch run while the
// preceding kernel of the stream drains; griddepcontrol.wait precedes the first
// access to global memory, and dependents are released after the last tile.
//
// Split-KV: when (batch x heads x query tiles) cannot fill the SMs, the key
// tiles of a query tile are split over 2, 4 or 8 CTAs that form a thread-block
// cluster.  After its last tile a CTA sends its rows' (max, sum) pairs to the
// peers with asynchronous stores that complete on the peers' mbarriers,
// stages its partial rows in shared memory (16-bit floats scaled by the row's
// largest magnitude, which travels with the row in fp32) and pushes each peer
// the rows that peer owns with one bulk copy; the owner weights the rows of all
// splits by exp2(m_split - m_row) / l_row and adds them in split order.  No
// cluster-wide barrier is on that path: peers signal each other through
// mbarriers, every wait is bounded.  Where clusters of that size cannot be
// scheduled the partials go through the caller's workspace instead (fp32) and
// the CTA that arrives last at a ticket counter merges them.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <stdlib.h>

#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace we {

constexpr int kBlockM = 128;    // queries per CTA (= TMEM lanes)
constexpr int kBlockN = 128;    // keys per tile
constexpr int kMaxTiles = 1024; // capacity limit: 131072 tokens per (row, head)
constexpr int kAttnThreads = 384;
constexpr int kSoftmaxThreads = 256;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0;    // + 128 * (tile & 1); group g owns columns [64g, 64g+64), P_g its first 32
constexpr uint32_t kColO = 256;  // + 128 * group
constexpr float kRescaleThreshold = 8.0f;  // log2 units
#ifndef WE_POLY_EVERY
#define WE_POLY_EVERY 4
#endif
// Every wait of the kernel goes through this macro; debug builds record the source line of a wait that gave up.
#ifdef WE_ATTN_DEBUG
#define WE_WAIT(...) mbar_wait(__VA_ARGS__, s_abort, kWaitLimitNs, kWaitMinPolls, __LINE__)
#else
#define WE_WAIT(...) mbar_wait(__VA_ARGS__, s_abort)
#endif
constexpr int kPolyEvery = WE_POLY_EVERY;  // one pair of exponentials in this many runs on the FMA pipe (0: none)

template <int DH>
struct AttnCfg {
  static constexpr int kChunks = DH / 64;                 // 128-byte column chunks per row
  static constexpr int kChunkBytes = kBlockN * 128;       // one chunk of a 128-row tile
  static constexpr int kTileBytes = kChunks * kChunkBytes;
  static constexpr int kStagesK = DH == 128 ? 3 : 4;      // stage counts also keep smem above half an SM,
  static constexpr int kStagesV = DH == 128 ? 2 : 4;      // so two CTAs never share an SM's tensor memory
  static constexpr int kSmemTiles = kTileBytes * (1 + kStagesK + kStagesV);
  static constexpr int kSmemAux = 64 * 8 + kMaxTiles * 2 + 64 + 4 * kBlockM * 4 + kMaxTiles + 8 * kBlockM * 8;
  static constexpr int kSmemBytes = kSmemTiles + kSmemAux + 1024;  // + slack for 1024-byte alignment
  // Exchange buffers of the epilogue, laid over the (then idle) rings: the CTA's partial O tile over the K ring,
  // the rows received from the other splits over the V ring.  A row travels as DH fp16 values, each half row
  // divided by its own largest magnitude, followed by 16 bytes that hold those two magnitudes as floats (the
  // 16 bytes also keep the row stride off a multiple of 128 bytes: no bank conflicts for 16-byte accesses).
  static constexpr int kPartRowB = DH * 2 + 16;
  static_assert(kBlockM * kPartRowB <= kStagesK * kTileBytes, "the partial tile must fit in the K ring");
  static_assert(kBlockM * kPartRowB <= kStagesV * kTileBytes,
                "the rows received from up to 7 peers (at most 7/8 of a tile) must fit in the V ring");
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
  int32_t ring_frames;           // L / T
  int32_t nsplit, n_qtiles;
  int32_t log2_nsplit;           // nsplit is a power of two
  int32_t gqa;                   // query heads per kv head
  int32_t hid_tiles_max;         // T / 128: the most whole key tiles a hidden slot can cover
  int32_t q_perm[3];             // which of (t, h, b) feeds tensor-map coordinate 1, 2, 3
  int32_t kv_perm[3];
  float scale_log2;
  float* ws_o;                   // [unit][split][DH][128]
  float* ws_ml;                  // [unit][split][2][128]
  int32_t* ws_cnt;               // [unit]
  int32_t* status;
  int32_t cluster_merge;         // 1: the splits of a query tile form a thread-block cluster and merge through DSMEM
  // fused append (we_b200_append_attend on tile-aligned caches): the tiles of the new frame are read from
  // k_new / v_new (tensor maps of their own) instead of the tail, and stored from shared memory into the cache
  // through the cache's tensor maps
  int32_t fused;
  int32_t is_frozen;
  int32_t kn_perm[3], vn_perm[3];
  uint8_t* written_w;
  // optional per-row output factor (the head gate of src/model/attn.py:117-119)
  const uint16_t* gate;
  int64_t gate_s[3];             // strides (b, h, t) in elements
  int32_t gate_logits;           // 1: apply sigmoid and round to the dtype first
};

#ifdef WE_ATTN_DEBUG
// Debug builds only: a per-CTA timeline (SM cycles since the CTA started) written to a caller-provided buffer.
__device__ uint32_t* g_trace = nullptr;
// Debug builds only: when set, the first CTA of an unsplit launch lets one wait run out on purpose -- a wait
// with a limit of a millisecond on a barrier nobody arrives on, before the CTA has issued a single copy or
// product -- and then goes on as any CTA does whose wait gave up: status word, teardown, tensor memory freed.
__device__ int g_expire_test = 0;
__device__ __forceinline__ long long trace_clock() {
  long long t;
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)::"memory");
  return t;
}
#define WE_TRACE(slot)                                                                             \
  do {                                                                                             \
    if (trace != nullptr) trace[(slot)] = static_cast<uint32_t>(trace_clock() - t_start);          \
  } while (0)
#define WE_TRACE_VAL(slot, val)                                                                    \
  do {                                                                                             \
    if (trace != nullptr) trace[(slot)] = static_cast<uint32_t>(val);                              \
  } while (0)
// Stamps inside the single-thread issue loops lengthen the very chain they measure: they are compiled in only
// on request (-DWE_ATTN_DEBUG_ISSUE).
#ifdef WE_ATTN_DEBUG_ISSUE
#define WE_TRACE_MMA(slot) WE_TRACE(slot)
constexpr bool kFullTrace = true;
#else
constexpr bool kFullTrace = false;     // per-tile stamps of the softmax warps too only on request: they cost time
#define WE_TRACE_MMA(slot) do {} while (0)
#endif
#else
constexpr bool kFullTrace = false;
#define WE_TRACE_MMA(slot) do {} while (0)
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

// a * wa + b * wb where a term with weight 0 is dropped outright (its value may be stale or non-finite)
__device__ __forceinline__ float merge2(float a, float wa, float b, float wb) {
  const float ta = wa != 0.f ? a * wa : 0.f;
  return wb != 0.f ? fmaf(b, wb, ta) : ta;
}

__device__ __forceinline__ void named_bar_arrive(int id, int nthreads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Packed fp32 pairs (Blackwell executes fma / add on two floats per instruction).
__device__ __forceinline__ uint64_t pk64(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void upk64(uint64_t v, uint32_t& lo, uint32_t& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t splat2(float x) { return pk64(__float_as_uint(x), __float_as_uint(x)); }
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void cluster_arrive_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
// Asynchronous bulk copy from this CTA's shared memory into a peer CTA's shared memory; completion is
// signalled as transaction bytes on the peer's mbarrier.  All addresses and the size are 16-byte multiples.
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster_addr, uint32_t src_cta_addr, uint32_t bytes,
                                                  uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          dst_cluster_addr),
      "r"(src_cta_addr), "r"(bytes), "r"(bar_cluster_addr)
      : "memory");
}
// Arrive (count 1) on an mbarrier in a peer CTA's shared memory.  Relaxed: it publishes no data, it only tells
// the peer that something it sent has been consumed.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// Asynchronous store of two floats into a peer CTA's shared memory; the 8 bytes are signalled on the peer's
// mbarrier as transaction bytes, so the data is visible to whoever sees that barrier phase complete.
__device__ __forceinline__ void st_async_f32x2(uint32_t dst_cluster_addr, float a, float b, uint32_t bar_cluster_addr) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];" ::"r"(
                   dst_cluster_addr),
               "f"(a), "f"(b), "r"(bar_cluster_addr)
               : "memory");
}

// Programmatic dependent launch: wait until the preceding kernel of the stream has completed and its
// writes are visible (returns at once when the launch carried no programmatic dependency).
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Is token `key` visible to this call?  (written, not in the hidden slot, inside the buffer.)
__device__ __forceinline__ bool token_visible(const uint8_t* wr, int key, int C, bool hide, int64_t slot_base, int T) {
  if (key >= C) return false;
  if (hide && key >= slot_base && key < slot_base + T) return false;
  return wr[key] != 0;
}

// Visibility bits of 32 consecutive tokens starting at key0 (partial tiles only; rare path).
__device__ __noinline__ uint32_t chunk_visibility(const uint8_t* wr, int key0, int C, bool hide, int64_t slot_base,
                                                  int T) {
  uint32_t bits = 0;
  for (int j = 0; j < 32; ++j) bits |= token_visible(wr, key0 + j, C, hide, slot_base, T) ? (1u << j) : 0u;
  return bits;
}

// slot_of() with a 32-bit fast path (frame counters below 2^31).
__device__ __forceinline__ void slot_of_fast(int64_t ft, int64_t L, int T, int dilation, int ring_frames, int& slot_base,
                                             int& hide) {
  if (static_cast<uint64_t>(ft) < 0x3FFFFFFFull) {
    const uint32_t t = static_cast<uint32_t>(ft), d = static_cast<uint32_t>(dilation);
    if (d == 1u) {                                  // the common case: one division instead of three
      slot_base = static_cast<int>((t % static_cast<uint32_t>(ring_frames)) * static_cast<uint32_t>(T));
      hide = 1;
    } else {
      const uint32_t buckets = static_cast<uint32_t>(ring_frames) / d;
      slot_base = static_cast<int>((((t + d - 1u) / d) % buckets) * static_cast<uint32_t>(T));
      hide = (t % d) == 0u;
    }
  } else {
    const SlotInfo si = slot_of(ft, L, T, dilation);
    slot_base = static_cast<int>(si.base);
    hide = si.write_step;
  }
}

// 16 bytes of `written` starting at token 16*v (zeros past the end of the buffer).
__device__ __forceinline__ uint4 load_written16(const uint8_t* wr, int v, int C) {
  uint4 w = make_uint4(0u, 0u, 0u, 0u);
  if (v * 16 + 16 <= C) {
    w = *reinterpret_cast<const uint4*>(wr + v * 16);
  } else if (v * 16 < C) {
    uint32_t ww[4] = {0u, 0u, 0u, 0u};
#pragma unroll 1
    for (int key = v * 16; key < C; ++key) {
      const uint32_t bit = (wr[key] != 0 ? 1u : 0u) << ((key & 3) * 8);
      const int word = (key & 15) >> 2;
      ww[0] |= word == 0 ? bit : 0u;
      ww[1] |= word == 1 ? bit : 0u;
      ww[2] |= word == 2 ? bit : 0u;
      ww[3] |= word == 3 ? bit : 0u;
    }
    w = make_uint4(ww[0], ww[1], ww[2], ww[3]);
  }
  return w;
}

template <int DH, bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 1)
frame_attn_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_kn,
                  const __grid_constant__ CUtensorMap tm_vn, const AttnParams p) {
  using Cfg = AttnCfg<DH>;
  constexpr int kStagesK = Cfg::kStagesK;
  constexpr int kStagesV = Cfg::kStagesV;
  constexpr uint32_t kInFmt = BF16 ? 1u : 0u;
  constexpr uint32_t kIdescS = umma_idesc(kInFmt, 0u, kBlockM, kBlockN);
  constexpr uint32_t kIdescPV = umma_idesc(kInFmt, 1u, kBlockM, DH);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::kTileBytes;
  uint8_t* sV = sK + kStagesK * Cfg::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kStagesV * Cfg::kTileBytes);
  uint64_t* q_full = bars + 0;
  uint64_t* recv_bar = bars + 1;  // incoming partial rows of the split merge
  uint64_t* ml_bar = bars + 2;    // peers: "my main loop is over and my (m, l) rows are in your table"
  uint64_t* ack_bar = bars + 3;   // peers: "the rows you pushed to me have landed"
  uint64_t* o_final = bars + 4;   // single phase: every MMA of the CTA complete
  uint64_t* p_ready = bars + 5;   // [tile & 1]: all eight softmax warps have written their share of P(tile)
  // One phase per load of the stage: S of the tile in K stage s is complete (the softmax warps may read it, the
  // producer may refill the stage) / both PV products of the tile in V stage s are complete (O may be touched,
  // the producer may refill the stage).  One commit of the issuing thread serves both kinds of waiter.
  uint64_t* s_ready = bars + 7;                 // [kStagesK]
  uint64_t* o_ready = s_ready + kStagesK;       // [kStagesV]
  uint64_t* k_full = o_ready + kStagesV;        // [kStagesK]
  uint64_t* v_full = k_full + kStagesK;         // [kStagesV]
  uint64_t* drained = v_full + kStagesV;        // single phase: the stages of unneeded early loads have been released
  uint16_t* s_list = reinterpret_cast<uint16_t*>(bars + 64);          // [kMaxTiles] (tile << 1) | partial
  uint32_t* s_misc = reinterpret_cast<uint32_t*>(s_list + kMaxTiles);
  uint32_t* s_tmem = s_misc + 0;
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_misc + 1);
  volatile uint32_t* s_nlist = s_misc + 2;
  uint32_t* s_ticket = s_misc + 12;
  volatile int64_t* s_slot = reinterpret_cast<volatile int64_t*>(s_misc + 4);  // [0] base, [1] hide flag
  float* s_ml = reinterpret_cast<float*>(s_misc + 16);                // [stream][m, l][128]
  float* s_x = s_ml;                                                  // [tile & 1][group][128] half-row exchange
  uint8_t* s_cnt = reinterpret_cast<uint8_t*>(s_ml + 4 * kBlockM);    // [kMaxTiles] visible keys per tile
  float* s_mltab = reinterpret_cast<float*>(s_cnt + kMaxTiles);       // [8 splits][128 rows][m, l]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int split = blockIdx.x & (p.nsplit - 1);   // consecutive blocks = the splits of one query tile (one cluster)
  const int qt = blockIdx.x >> p.log2_nsplit;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int kvh = p.gqa == 1 ? h : h / p.gqa;
  const int q0 = qt * kBlockM;
  const uint8_t* wr = p.written + static_cast<int64_t>(b) * p.written_batch_stride;
  // Factor of output row `r` of this tile: 1, or the head gate (sigmoid of the logit, rounded to the tensors'
  // dtype as the reference's `gates` tensor is, src/model/attn.py:117-119).
  auto row_gate = [&](int r) -> float {
    if (p.gate == nullptr || q0 + r >= p.T) return 1.f;
    const uint16_t raw = p.gate[b * p.gate_s[0] + h * p.gate_s[1] + static_cast<int64_t>(q0 + r) * p.gate_s[2]];
    float gv = BF16 ? __uint_as_float(static_cast<uint32_t>(raw) << 16) : __half2float(__ushort_as_half(raw));
    if (p.gate_logits) {
      gv = 1.0f / (1.0f + expf(-gv));
      gv = BF16 ? __bfloat162float(__float2bfloat16_rn(gv)) : __half2float(__float2half_rn(gv));
    }
    return gv;
  };
#ifdef WE_ATTN_DEBUG
  const long long t_start = trace_clock();
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

  // One K or V tile into a ring stage.  With the fused append the tiles of the tail frame come straight from
  // k_new / v_new (the copy into the cache happens on the side and is never read back in this launch).
  // (coordinates are routed to the tensor map's axes with selects: an indexed array would live in local memory)
  auto pick3 = [](int which, int a0, int a1, int a2) { return which == 0 ? a0 : (which == 1 ? a1 : a2); };
  auto load_kv_tile = [&](bool is_k, uint8_t* dst, uint64_t* bar, int key0) {
    const bool from_new = p.fused && key0 >= p.L;
    const CUtensorMap* tm = is_k ? (from_new ? &tm_kn : &tm_k) : (from_new ? &tm_vn : &tm_v);
    const int32_t* perm = from_new ? (is_k ? p.kn_perm : p.vn_perm) : p.kv_perm;
    const int tok = from_new ? key0 - static_cast<int>(p.L) : key0;
    const int x1 = pick3(perm[0], tok, kvh, b), x2 = pick3(perm[1], tok, kvh, b), x3 = pick3(perm[2], tok, kvh, b);
    mbar_arrive_expect_tx(bar, Cfg::kTileBytes);
#pragma unroll
    for (int ch = 0; ch < Cfg::kChunks; ++ch) tma_load_4d(dst + ch * Cfg::kChunkBytes, tm, bar, ch * 64, x1, x2, x3);
  };

  // With the fused append the tiles of the new frame are also persisted (LayerKVCache.upsert,
  // src/model/kv_cache.py:138,147-150): each of them, K and V, goes into the tail slice and, on an unfrozen write
  // step, into the ring slot: "jobs" of one tensor store each (the stores un-swizzle on the way out, like the
  // loads swizzled).  A tensor store is slow to issue (measured: a quarter of a microsecond per 16 KB box, during
  // which the issuing thread and the loads queued behind it wait), so the jobs are dealt out among ALL CTAs
  // that work for the kv head (every split of every query tile and query head sharing it), one or two each, and
  // a CTA does its jobs when its K producer has requested the last tile of the walk and would idle: it fetches
  // the new tile once more (from L2) into the K-ring stage that frees up next and stores it from there.
  // Nothing in this launch reads the places written (the tail tiles are read from k_new / v_new, the slot is
  // hidden), so the order against the other CTAs does not matter.
  const int n_sharers = p.n_qtiles * p.gqa;
  const int job_first = split * n_sharers + qt * p.gqa + (h - kvh * p.gqa);
  const int job_step = p.nsplit * n_sharers;
  auto store_new_tile = [&](bool is_k, const uint8_t* src, int tile, bool into_slot, int slot_base) {
    const CUtensorMap* tm = is_k ? &tm_k : &tm_v;
    const int tok = (into_slot ? slot_base : static_cast<int>(p.L)) + tile * kBlockN;
    const int x1 = pick3(p.kv_perm[0], tok, kvh, b), x2 = pick3(p.kv_perm[1], tok, kvh, b),
              x3 = pick3(p.kv_perm[2], tok, kvh, b);
#pragma unroll
    for (int ch = 0; ch < Cfg::kChunks; ++ch) tma_store_4d(tm, src + ch * Cfg::kChunkBytes, ch * 64, x1, x2, x3);
  };

  // ---------------------------------------------------------------- set-up
  // On-chip part first: it needs nothing from global memory, so it may run while the preceding kernel of the
  // stream is still finishing (programmatic dependent launch).
  if (warp == 8) {
    // (the abort word is cleared by the warp that is first to wait on a barrier; the others read it only after
    // the set-up barrier below)
    if (lane == 0) *s_abort = 0;
    // one barrier per lane: [0] q_full [1] recv_bar [2] ml_bar [3] ack_bar [4] o_final [5,6] p_ready, then
    // s_ready, o_ready, k_full, v_full, drained
    constexpr int kNumBars = 8 + 2 * (kStagesK + kStagesV);
    static_assert(kNumBars <= 32, "one lane per barrier");
    if (lane < kNumBars) {
      const int peers = p.nsplit > 1 ? p.nsplit - 1 : 1;
      mbar_init(bars + lane, (lane == 5 || lane == 6) ? 8 : (lane == 3 ? peers : 1));   // p_ready: one arrival per warp
    }
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      if (p.fused) {
        prefetch_tensormap(&tm_kn);
        prefetch_tensormap(&tm_vn);
      }
    }
    __syncwarp();
    if (lane == 0) {
      fence_mbar_init();
      fence_proxy_async_smem();
      if (p.cluster_merge && p.nsplit > 1) {
        // bytes the peers will send to this CTA at the end: their (m, l) pairs and the weighted rows it owns
        const int rows_mine = kBlockM >> p.log2_nsplit;
        mbar_arrive_expect_tx(ml_bar, static_cast<uint32_t>((p.nsplit - 1) * kBlockM * 8));
        mbar_arrive_expect_tx(recv_bar, static_cast<uint32_t>((p.nsplit - 1) * rows_mine * Cfg::kPartRowB));
      }
    }
    __syncwarp();
#ifdef WE_ATTN_DEBUG
    if (lane == 0 && p.nsplit == 1 && blockIdx.x + blockIdx.y + blockIdx.z == 0 && g_expire_test != 0)
      mbar_wait(ack_bar, 0, s_abort, 1000ull * 1000ull, 64u, __LINE__);   // (no split: nobody ever arrives on it)
#endif
    named_bar_arrive(4, kAttnThreads);
  }
  if (warp == 9) {
    tmem_alloc(s_tmem, kTmemCols);
    tmem_relinquish();
    if (lane == 0) WE_TRACE(8);
  }
  // Everything below reads global memory that the preceding kernel of the stream may have produced (the
  // queries, the new rows, the cache, the frame counter): wait until that kernel has completed and its writes
  // are visible.  Returns at once when the launch carried no programmatic dependency.
  if (tid == 0) WE_TRACE(4);
  grid_dependency_wait();
  if (tid == 0) WE_TRACE(5);
  const int64_t ft = p.frame_t[static_cast<int64_t>(b) * p.frame_t_stride];
  if (warp == 8 && lane == 0) {
    // Q tile: rows q0 .. q0+127 of (b, h); rows past T are zero-filled by TMA.  It does not depend on the frame
    // counter, so it goes out while that load is in flight.
    mbar_arrive_expect_tx(q_full, Cfg::kTileBytes);
    const int x1 = pick3(p.q_perm[0], q0, h, b), x2 = pick3(p.q_perm[1], q0, h, b), x3 = pick3(p.q_perm[2], q0, h, b);
#pragma unroll
    for (int ch = 0; ch < Cfg::kChunks; ++ch) tma_load_4d(sQ + ch * Cfg::kChunkBytes, &tm_q, q_full, ch * 64, x1, x2, x3);
  }
  // The visibility scan is done by every warp but the producer (warp 8), which fetches tiles meanwhile.  Its loads
  // of `written` go out before the frame counter is known, for every physical tile this CTA can possibly be
  // given: candidate ranges move by at most the tiles of one hidden slot.
  constexpr int kScanThreads = kAttnThreads - 32;
  const int stid = tid < 256 ? tid : tid - 32;
  const int c0_min = ((p.ntiles - p.hid_tiles_max) * split) >> p.log2_nsplit;
  int span = ((p.ntiles * (split + 1)) >> p.log2_nsplit) + p.hid_tiles_max - c0_min;
  span = min(span, p.ntiles - c0_min);
  const int my_j = stid >> 3;
  const uint4 w_first = load_written16(wr, my_j < span ? (c0_min + my_j) * 8 + (stid & 7) : 0x3FFFFFF, p.C);
  // Candidate tiles = physical tiles minus those that lie entirely in the hidden slot (pure arithmetic on
  // the frame counter).  Split `split` owns candidates [c0, c1); which of them hold a visible key is decided
  // below from `written`.
  int slot_base, hide_i;
  slot_of_fast(ft, p.L, p.T, p.dilation, p.ring_frames, slot_base, hide_i);
  if (tid == 0) WE_TRACE(6 + (slot_base & 0));
  const int hid_lo = hide_i ? slot_base : 0, hid_hi = hide_i ? slot_base + p.T : 0;   // hidden token range
  const int first_h = hide_i ? (slot_base + kBlockN - 1) / kBlockN : 0;
  const int last_h = hide_i ? (slot_base + p.T) / kBlockN : 0;
  const int count_h = last_h > first_h ? last_h - first_h : 0;
  const int n_cand = p.ntiles - count_h;
  const int c0 = (n_cand * split) >> p.log2_nsplit;
  const int c1 = (n_cand * (split + 1)) >> p.log2_nsplit;
  const int np = c1 - c0;
  auto phys_tile = [&](int c) { return c < first_h ? c : c + count_h; };
  // Order in which this CTA walks its candidates: the tiles of the tail frame first (only the last split has
  // them).  They were written by the kernel just ahead (or come from k_new / v_new), so they arrive from L2
  // rather than from DRAM and the first product starts sooner.  (The order of the tiles does not matter to the
  // result beyond the rounding of the running sums.)
  const int c_tail = (p.L % kBlockN == 0) ? static_cast<int>(p.L / kBlockN) - count_h : n_cand;
  const int n_tail = max(0, c1 - max(c0, c_tail));
  auto cand_tile = [&](int j) { return phys_tile(c0 + (j < n_tail ? np - n_tail + j : j - n_tail)); };
  constexpr int kBlind = 2;                       // tiles loaded before their visibility is known
  const int nblind = np < kBlind ? np : kBlind;
  if (warp == 8 && lane == 0) {
    // The first tiles of the range, before it is known whether they hold a visible key (they almost always
    // do; a miss is drained later): DRAM latency then overlaps the rest of the set-up and the scan.  K(0),
    // which the first product needs, goes first.
    WE_TRACE(11);
    if (nblind > 0) load_kv_tile(true, sK, &k_full[0], cand_tile(0) * kBlockN);
    WE_TRACE(12);
    if (nblind > 0) load_kv_tile(false, sV, &v_full[0], cand_tile(0) * kBlockN);
    for (int j = 1; j < nblind; ++j) {
      const int key0 = cand_tile(j) * kBlockN;
      load_kv_tile(true, sK + j * Cfg::kTileBytes, &k_full[j], key0);
      load_kv_tile(false, sV + j * Cfg::kTileBytes, &v_full[j], key0);
    }
    WE_TRACE(7);
  }
  // Set-up barrier.  The producer warp only arrives (it did so above, right after initialising the mbarriers):
  // it needs nothing from the other warps and goes on issuing loads.
  if (warp != 8) {
    tc_fence_before();
    named_bar_sync(4, kAttnThreads);
    tc_fence_after();
  }
  // Split-phase cluster barrier: "my barriers are initialised" now, awaited much later, right before the
  // first access to a peer's shared memory.
  // (relaxed: the barrier initialisation was already published by fence.mbarrier_init.release.cluster)
  if (p.cluster_merge && p.nsplit > 1) cluster_arrive_relaxed();
  if (tid == 0) WE_TRACE(1);
  const uint32_t tmem_base = *s_tmem;

  // ------------------------------------------------------ visible-tile list
  // While the first tiles are on their way, all warps but the producer scan `written`: 16 tokens per thread,
  // eight lanes make one 128-key tile; warp 11 compacts the per-tile counts into the list of tiles to walk.
  int n = 0;                 // tiles of this CTA with at least one visible key
  uint32_t blind_vis = 0;    // bit j: the j-th tile loaded ahead of time turned out visible
  if (warp != 8) {
    if (stid == 0) {
      s_slot[0] = slot_base;
      s_slot[1] = hide_i;
    }
    const int nvec_pad = (span * 8 + 31) & ~31;    // whole warps take part in the shuffles
#pragma unroll 1
    for (int idx = stid; idx < nvec_pad; idx += kScanThreads) {
      const int j = idx >> 3;                        // physical tile c0_min + j
      const int v = j < span ? (c0_min + j) * 8 + (idx & 7) : 0x3FFFFFF;
      uint4 w = w_first;
      if (idx != stid) w = load_written16(wr, v, p.C);
      const int k0 = v * 16;
      // one bit per non-zero byte
      const uint32_t nz0 = __vcmpne4(w.x, 0u) & 0x01010101u, nz1 = __vcmpne4(w.y, 0u) & 0x01010101u;
      const uint32_t nz2 = __vcmpne4(w.z, 0u) & 0x01010101u, nz3 = __vcmpne4(w.w, 0u) & 0x01010101u;
      int cnt = __popc(nz0) + __popc(nz1) + __popc(nz2) + __popc(nz3);
      const int lo = max(k0, hid_lo), hi = min(k0 + 16, hid_hi);
      if (j < span && lo < hi) {
        if (lo == k0 && hi == k0 + 16) {
          cnt = 0;                                   // the whole vector lies in the hidden slot
        } else {
#pragma unroll 1
          for (int key = lo; key < hi; ++key) cnt -= (key < p.C && wr[key] != 0) ? 1 : 0;
        }
      }
      cnt += __shfl_xor_sync(0xffffffffu, cnt, 1);
      cnt += __shfl_xor_sync(0xffffffffu, cnt, 2);
      cnt += __shfl_xor_sync(0xffffffffu, cnt, 4);
      if ((lane & 7) == 0 && j < span) s_cnt[j] = static_cast<uint8_t>(cnt);
    }
    named_bar_sync(3, kScanThreads);
    if (warp == 11) {
#pragma unroll 1
      for (int base = 0; base < np; base += 32) {
        const int j = base + lane;
        const int c = j < np ? s_cnt[cand_tile(j) - c0_min] : 0;
        const unsigned m = __ballot_sync(0xffffffffu, c != 0);
        if (c != 0)
          s_list[n + __popc(m & ((1u << lane) - 1u))] =
              static_cast<uint16_t>((cand_tile(j) << 1) | (c != kBlockN ? 1 : 0));
        if (base == 0) blind_vis = m & ((1u << nblind) - 1u);
        n += __popc(m);
      }
      if (lane == 0) {
        s_nlist[0] = static_cast<uint32_t>(n);
        s_nlist[1] = blind_vis;
      }
      __threadfence_block();
    }
  }
  if (warp == 11) {
    named_bar_arrive(2, kAttnThreads);   // the other warps sleep on this barrier instead of polling
  } else {
    named_bar_sync(2, kAttnThreads);
    n = static_cast<int>(s_nlist[0]);
    blind_vis = s_nlist[1];
  }
  constexpr int t0 = 0;
  // Position of the i-th visible tile in the order the tiles were (or will be) loaded: the tiles fetched ahead
  // of time come first, whether visible or not; every later load is a visible tile.
  const int n_vis_blind = __popc(blind_vis);
  auto load_seq = [&](int i) {
    if (i < n_vis_blind) return (i == 0 && (blind_vis & 1u)) ? 0 : 1;   // kBlind == 2
    return i + (nblind - n_vis_blind);
  };
  if (tid == 0) { WE_TRACE(2); WE_TRACE_VAL(3, n); WE_TRACE_VAL(231, blind_vis | (nblind << 8) | (np << 16)); }

  // Tensor products of the tiles of one parity (thread 0 of warp 9: even tiles, of warp 11: odd tiles):
  //   S(i) = Q K(i)^T      M=128 queries, N=128 keys, K=DH in steps of 16, both operands in shared memory
  //                        (K-major, 128-byte swizzle), into S buffer i & 1;
  //   O_g += P_g(i) V_g(i) for the two key halves g: M=128, N=DH, K=64 keys in steps of 16; P_g sits in the first
  //                        32 columns of group g's half of S(i) (two 16-bit values per column), V is read from
  //                        shared memory as an MN-major operand.
  // A thread issues S(p), then for its tiles i: P V(i) followed at once by S(i+2), which overwrites the columns of
  // P(i): products of one thread execute in the order issued, so no barrier is needed between the two.  Issuing a
  // product blocks the thread for about as long as the tensor pipe needs for it; with two issuing threads the
  // waits and commits of one overlap the products of the other.  P V(i) and P V(i-1) add into the same
  // accumulators from different threads: the later one waits for the earlier one's completion barrier.
  auto issue_products = [&](int parity) {
    const uint32_t q_lo = umma_desc_lo(smem_u32(sQ), 16);                       // K-major, 128-byte swizzle
    const uint32_t k_lo = umma_desc_lo(smem_u32(sK), 16);
    const uint32_t v_lo = umma_desc_lo(smem_u32(sV), Cfg::kChunkBytes);         // MN-major: LBO = chunk stride
    constexpr uint32_t kTileStep = Cfg::kTileBytes >> 4;
    auto issue_s = [&](int i) {
      const int a = load_seq(i);
      const int sk = a % kStagesK;
      WE_WAIT(&k_full[sk], (a / kStagesK) & 1);
      const uint32_t d = tmem_base + kColS + 128u * (i & 1);
      const uint32_t kb = k_lo + sk * kTileStep;
      umma_ss_lo<0>(d, q_lo, kb, kIdescS);
#pragma unroll
      for (int kk = 1; kk < DH / 16; ++kk) {
        constexpr uint32_t kChunkStep = Cfg::kChunkBytes >> 4;
        const uint32_t off = (kk >> 2) * kChunkStep + (kk & 3) * 2;          // 32 bytes per K step
        umma_ss_lo<1>(d, q_lo + off, kb + off, kIdescS);
      }
      tc_commit(&s_ready[sk]);        // the softmax warps are waiting for this one; it also frees the K stage
    };
    WE_TRACE_VAL(210 + parity, 900);
    if (parity != 0) WE_WAIT(drained, 0);
    WE_WAIT(q_full, 0);
    WE_TRACE_VAL(210 + parity, 901);
    if (parity == 0) WE_TRACE(13);
    if (parity == 0) { WE_WAIT(&k_full[load_seq(0) % kStagesK], 0); WE_TRACE(14); }
    issue_s(parity);
    if (parity == 0) WE_TRACE(15);
    for (int i = parity; i < n; i += 2) {
      const int av = load_seq(i);
      const int sv = av % kStagesV;
      const int buf = i & 1;
      // everything that is ready long before P(i) is waited for first
      WE_TRACE_VAL(210 + parity, 1000 + 10 * i + 1);
      WE_WAIT(&v_full[sv], (av / kStagesV) & 1);
      WE_TRACE_VAL(210 + parity, 1000 + 10 * i + 2);
      if (i + 2 < n) {
        const int a2 = load_seq(i + 2);
        WE_WAIT(&k_full[a2 % kStagesK], (a2 / kStagesK) & 1);
      }
      WE_TRACE_VAL(210 + parity, 1000 + 10 * i + 3);
      if (i > 0) {
        const int ap = load_seq(i - 1);
        WE_WAIT(&o_ready[ap % kStagesV], (ap / kStagesV) & 1);
      }
      if (i == 4 || i == 5) WE_TRACE(180 + 8 * (i - 4));
      WE_TRACE_VAL(210 + parity, 1000 + 10 * i + 4);
      WE_WAIT(&p_ready[buf], (i >> 1) & 1);
      WE_TRACE_VAL(210 + parity, 1000 + 10 * i + 5);
      if (i == 4 || i == 5) WE_TRACE(181 + 8 * (i - 4));
      tc_fence_after();
      const uint32_t vb = v_lo + sv * kTileStep;
      const uint32_t acc0 = i > 0 ? 1u : 0u;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const uint32_t d = tmem_base + kColO + 128u * g;
        const uint32_t a_t = tmem_base + kColS + 128u * buf + 64u * g;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)                                          // 16 keys = 2048 bytes of V rows
          umma_ts_lo(d, a_t + kk * 8, vb + ((64 * g + 16 * kk) * 128 >> 4), kIdescPV, kk == 0 ? acc0 : 1u);
      }
      tc_commit(&o_ready[sv]);        // O may be touched again, and the V stage is free
      if (i == 4 || i == 5) WE_TRACE(182 + 8 * (i - 4));
      if (i + 2 < n) issue_s(i + 2);
      if (i == 4 || i == 5) WE_TRACE(183 + 8 * (i - 4));
      if (i == n - 1) tc_commit(o_final);
    }
  };

  // ------------------------------------------------------------------ roles
  if (warp == 8 || warp == 10) {
    // Producers: warp 8 feeds the K ring, warp 10 the V ring (a ring of its own, so that a full V ring never
    // holds back a K load).  A tile is issued as soon as the product that used its stage has completed.
    if (lane == 0) {
      const bool is_k = warp == 8;
      uint8_t* ring = is_k ? sK : sV;
      uint64_t* full = is_k ? k_full : v_full;
      uint64_t* empty = is_k ? s_ready : o_ready;
      const int stages = is_k ? kStagesK : kStagesV;
      const int nloads = nblind + n - n_vis_blind;
      auto key_of = [&](int a) {
        return (a < nblind ? cand_tile(a) : (s_list[a - nblind + n_vis_blind] >> 1)) * kBlockN;
      };
      for (int a = nblind; a < nloads; ++a) {
        const int st = a % stages;
        WE_TRACE_VAL(208 + (is_k ? 0 : 1), 100 + a);
        if (a >= stages) WE_WAIT(&empty[st], ((a / stages) - 1) & 1);
        if (is_k && a - nblind < 32) WE_TRACE_MMA(192 + a - nblind);
        load_kv_tile(is_k, ring + st * Cfg::kTileBytes, &full[st], key_of(a));
      }
      if (is_k && p.fused) {
        // this CTA's share of the store jobs: job = (K or V) + 2 * (tile + tiles * (tail or slot))
        const int tiles = p.T / kBlockN;
        const int n_jobs = 2 * tiles * ((!p.is_frozen && hide_i) ? 2 : 1);
        int a = nloads;                                  // the ring goes on with loads that no product consumes
        for (int job = job_first; job < n_jobs; job += job_step, ++a) {
          const bool k_plane = (job & 1) == 0;
          const int tile = (job >> 1) % tiles;
          const bool into_slot = (job >> 1) >= tiles;
          const int st = a % stages;
          // the stage is free when the product that read its last tile is complete, or, when an earlier job of
          // this loop used it (more jobs than stages), when that job's store has read it
          if (a >= stages && a - stages < nloads && !WE_WAIT(&empty[st], ((a / stages) - 1) & 1)) break;
          if (a - stages >= nloads) bulk_wait_group_read0();
          load_kv_tile(k_plane, ring + st * Cfg::kTileBytes, &full[st], static_cast<int>(p.L) + tile * kBlockN);
          if (!WE_WAIT(&full[st], (a / stages) & 1)) break;             // giving up: store nothing
          store_new_tile(k_plane, ring + st * Cfg::kTileBytes, tile, into_slot, slot_base);
          bulk_commit_group();
        }
        bulk_wait_group_read0();
      }
      if (is_k && n == 0) WE_WAIT(q_full, 0);  // nobody else consumes Q: let the copy land before exit
    }
    __syncwarp();
    // the rings are no longer read by stores of this warp: the epilogue may lay its exchange buffers over them
    named_bar_arrive(5, kSoftmaxThreads + 64);
    if (lane == 0 && p.fused) bulk_wait_group0();  // global writes performed before the CTA can exit
  } else if (warp == 9) {
    if (lane == 0) {
      // tiles fetched ahead of time that hold no visible key: let them land, then free their stages
      for (int j = 0; j < nblind; ++j) {
        if (!((blind_vis >> j) & 1u)) {
          WE_TRACE_VAL(210, 1 + 10 * j);
          WE_WAIT(&k_full[j], 0);
          mbar_arrive(&s_ready[j]);
          WE_TRACE_VAL(210, 2 + 10 * j);
          WE_WAIT(&v_full[j], 0);
          mbar_arrive(&o_ready[j]);
          WE_TRACE_VAL(210, 3 + 10 * j);
        }
      }
      // The other issuing thread waits for this before its first barrier wait: a wait for the second phase of a
      // stage barrier would pass at once while that barrier is still in its first phase (the early load has not
      // landed yet), and the product issued on it would then complete the phase that belongs to the release
      // above.
      mbar_arrive(drained);
    }
    if (lane == 0 && n > 0) issue_products(0);
    __syncwarp();
  } else if (warp < 8) {
    // ------------------------------------------------------- softmax warps
    // Both groups own all 128 rows.  Group g handles keys [64g, 64g+64) of every tile as a stream of its own:
    // own running maximum, own row sum, own accumulator O_g, so the groups never exchange data per tile.
    const int wg = warp >> 2;
    const int row = tid & 127;           // query row within the tile == TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    constexpr int kHalf = DH / 2;
    const int col0 = wg * kHalf;
    const uint32_t o_mine = tmem_base + lane_base + kColO + 128u * wg;
    const int slot_base = static_cast<int>(s_slot[0]);
    const bool hide = s_slot[1] != 0;
    float m_run = -INFINITY;  // running row maximum, log2 domain, possibly stale by <= threshold
    float l_run = 0.f;        // row sum over this group's keys
    // Second half of the split-phase cluster barrier (every CTA of the cluster has initialised its mbarriers),
    // needed before the first access to a peer's shared memory after the loop; by now it completes at once.
    if (p.cluster_merge && p.nsplit > 1) cluster_wait_acquire();
    for (int i = 0; i < n; ++i) {
      const int buf = i & 1;
      const uint32_t s_addr = tmem_base + lane_base + kColS + 128u * buf + 64u * wg;
      const int a_i = load_seq(i);
      if (row == 0) WE_TRACE_VAL(212 + wg, 10 * i + 1);
      WE_WAIT(&s_ready[a_i % kStagesK], (a_i / kStagesK) & 1);
      if (row == 0) WE_TRACE_VAL(212 + wg, 10 * i + 2);
      if (row == 0 && i < 32 && (kFullTrace || i == 1 || i == 4 || i == 5 || i == n - 1)) WE_TRACE(16 + 4 * i + 2 * wg);
      tc_fence_after();
      uint32_t s[2][32];
      tmem_ld32(s_addr, s[0]);
      tmem_ld32(s_addr + 32, s[1]);
      tmem_ld_wait();
      if (row == 0 && i == 4) WE_TRACE(200 + 4 * wg + 0);
      if (kFullTrace && row == 0 && i == 3) WE_TRACE(160 + 8 * wg + 0);
      const uint32_t entry = s_list[t0 + i];
      if (entry & 1u) {
        // partial tile: mask tokens that are unwritten, hidden, or beyond the buffer
        const int key0 = static_cast<int>(entry >> 1) * kBlockN + 64 * wg;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const uint32_t vis = chunk_visibility(wr, key0 + c * 32, p.C, hide, slot_base, p.T);
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (!((vis >> e) & 1u)) s[c][e] = 0xFF800000u;  // -inf
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int e = 0; e < 32; e += 8) {      // three-input max: two elements per instruction, four chains
          mx4[0] = max3(mx4[0], __uint_as_float(s[c][e + 0]), __uint_as_float(s[c][e + 1]));
          mx4[1] = max3(mx4[1], __uint_as_float(s[c][e + 2]), __uint_as_float(s[c][e + 3]));
          mx4[2] = max3(mx4[2], __uint_as_float(s[c][e + 4]), __uint_as_float(s[c][e + 5]));
          mx4[3] = max3(mx4[3], __uint_as_float(s[c][e + 6]), __uint_as_float(s[c][e + 7]));
        }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // A half tile may be fully masked (its visible keys all lie in the other half): keep the maximum finite
      // so that exp2(-inf - m) stays 0 instead of NaN.
      const float m_new = fmaxf(fmaxf(m_run, mx * p.scale_log2), -1e30f);
      const bool need = (m_new - m_run) > kRescaleThreshold;  // first tile: inf > threshold
      float alpha = 1.f;
      const bool raise = __any_sync(0xffffffffu, need);
      if (raise) {
        alpha = fast_exp2(m_run - m_new);                       // first tile: exp2(-inf) = 0
        l_run *= alpha;
        m_run = m_new;
      }
      // P = exp2(S * scale - m): the argument on packed fp32 pairs (one FMA per pair).  The special-function
      // pipe (16 ex2 per clock and SM) is what bounds this loop, so one pair in kPolyEvery is evaluated on the
      // FMA pipe instead: round to the nearest integer n with the 1.5 * 2^23 trick, a cubic in x - n (relative
      // error 7.5e-5, far below the rounding of P to 16 bits), n added into the exponent field.  Tiles with
      // masked keys (scores of -inf) take the special-function pipe for every element.
      if (row == 0 && i == 4) WE_TRACE(200 + 4 * wg + 1);
      const uint64_t scale2 = splat2(p.scale_log2), negm2 = splat2(-m_run);
      uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};
      uint32_t pk[32];
      auto exponentials = [&](auto poly_c) {
        constexpr bool kPoly = decltype(poly_c)::value;
        const uint64_t magic2 = splat2(12582912.f), nmagic2 = splat2(-12582912.f), mone2 = splat2(-1.f);
        const uint64_t c0 = splat2(0.9999280571937561f), c1 = splat2(0.6932609677314758f),
                       c2 = splat2(0.2426111251115799f), c3 = splat2(0.05517164617776871f);
#pragma unroll
        for (int q = 0; q < 32; ++q) {
          const int c = q >> 4, e = q & 15;
          const uint64_t x2 = fma2(pk64(s[c][2 * e], s[c][2 * e + 1]), scale2, negm2);
          uint32_t pl, ph;
          if (kPoly && kPolyEvery > 0 && (q % (kPolyEvery > 0 ? kPolyEvery : 1)) == (kPolyEvery > 0 ? kPolyEvery : 1) - 1) {
            const uint64_t t2 = add2(x2, magic2);
            const uint64_t n2 = add2(t2, nmagic2);
            const uint64_t f2 = fma2(n2, mone2, x2);
            uint64_t p2 = fma2(c3, f2, c2);
            p2 = fma2(p2, f2, c1);
            p2 = fma2(p2, f2, c0);
            uint32_t tl, th;
            upk64(t2, tl, th);
            upk64(p2, pl, ph);
            // exponent: n >= -126 (as integers the bit patterns of t order like the values; t < 0 reads negative)
            constexpr int kMinT = 0x4B400000 - 126;
            pl += static_cast<uint32_t>(max(static_cast<int>(tl), kMinT)) << 23;
            ph += static_cast<uint32_t>(max(static_cast<int>(th), kMinT)) << 23;
          } else {
            uint32_t xl, xh;
            upk64(x2, xl, xh);
            pl = __float_as_uint(fast_exp2(__uint_as_float(xl)));
            ph = __float_as_uint(fast_exp2(__uint_as_float(xh)));
          }
          sum2[q & 3] = add2(sum2[q & 3], pk64(pl, ph));
          pk[q] = pack2<BF16>(__uint_as_float(pl), __uint_as_float(ph));
        }
      };
      if (entry & 1u) exponentials(std::false_type{});
      else exponentials(std::true_type{});
      if (row == 0 && i == 4) WE_TRACE(200 + 4 * wg + 2);
      float sum4[4];
      {
        const uint64_t t01 = add2(sum2[0], sum2[1]), t23 = add2(sum2[2], sum2[3]);
        uint32_t a0, a1, b0, b1;
        upk64(t01, a0, a1);
        upk64(t23, b0, b1);
        sum4[0] = __uint_as_float(a0);
        sum4[1] = __uint_as_float(a1);
        sum4[2] = __uint_as_float(b0);
        sum4[3] = __uint_as_float(b1);
      }
      tmem_st32(s_addr, pk);                                    // P over the S columns this thread has consumed
      l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      if (kFullTrace && row == 0 && i < 32) WE_TRACE(17 + 4 * i + 2 * wg);
      if (i > 0 && raise) {
        // O_g is rescaled in place: PV(i-1) must have completed.  (Waiting only here is safe: the phase after
        // this one on the same barrier belongs to PV(i+1), which cannot complete before P(i+1) exists.)
        const int a_p = load_seq(i - 1);
        WE_WAIT(&o_ready[a_p % kStagesV], (a_p / kStagesV) & 1);
        {
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < DH / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(o_mine + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st32(o_mine + c * 32, o);
          }
        }
      }
      tmem_st_wait();
      if (row == 0 && i == 4) WE_TRACE(200 + 4 * wg + 3);
      if (kFullTrace && row == 0 && i == 3) WE_TRACE(160 + 8 * wg + 6);
      tc_fence_before();
      // one arrival per warp: 128 separate arrivals on one barrier word would queue up behind one another
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[buf]);
      if (kFullTrace && row == 0 && i == 3) WE_TRACE(160 + 8 * wg + 7);
    }

    // ---------------------------------------------------------- after the last tile
    // A kernel queued behind this one with a programmatic dependency (the next layer-step's append) may be
    // scheduled from here on; it waits for this grid to complete before it touches memory.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (n > 0) {
      WE_WAIT(o_final, 0);   // (the per-tile barriers of the other group were never followed here)
      tc_fence_after();
    }
    if (row == 0) WE_TRACE(224 + wg);
    // merge the two groups' streams: exchange (m, l); each group then combines one half of the head dim.  The
    // barrier of the exchange is also the one the producer warps arrive on when they are done with the rings
    // (tensor stores of new-frame tiles have read them).
    s_x[(wg * 2 + 0) * kBlockM + row] = m_run;
    s_x[(wg * 2 + 1) * kBlockM + row] = l_run;
    named_bar_sync(5, kSoftmaxThreads + 64);
    const float m_oth = s_x[((wg ^ 1) * 2 + 0) * kBlockM + row];
    const float l_oth = s_x[((wg ^ 1) * 2 + 1) * kBlockM + row];
    const float m_cta = fmaxf(m_run, m_oth);                       // -inf when the split got no tile
    const float w_mine = l_run > 0.f ? fast_exp2(m_run - m_cta) : 0.f;
    const float w_oth = l_oth > 0.f ? fast_exp2(m_oth - m_cta) : 0.f;
    const float l_cta = l_run * w_mine + l_oth * w_oth;            // 0 when the split got no tile
    const float w_g0 = wg == 0 ? w_mine : w_oth, w_g1 = wg == 0 ? w_oth : w_mine;
    const uint32_t o0_addr = tmem_base + lane_base + kColO + col0;   // this thread's column half of O_0
    const uint32_t o1_addr = o0_addr + 128u;                          // ... and of O_1
    const bool in_range = q0 + row < p.T;
    uint8_t* orow = static_cast<uint8_t*>(p.out) +
                    2 * (b * p.os[0] + h * p.os[1] + static_cast<int64_t>(q0 + row) * p.os[2] + col0);
    if (p.cluster_merge) {
      float wgt = 1.0f;
      if (p.nsplit == 1) {
        wgt = (1.0f / l_cta) * row_gate(row);
      } else {
        // every CTA of the cluster learns every split's (m, l): group 0 sends its rows' pair to all peers as
        // asynchronous stores that complete on the peer's barrier (no fence, no extra arrival).  The pairs
        // are consumed only when the rows are summed, so their flight overlaps the staging below.
        if (wg == 0) {
          const uint32_t mine = smem_u32(s_mltab + (split * kBlockM + row) * 2);
          const uint32_t bar = smem_u32(ml_bar);
          for (int d = 0; d < p.nsplit; ++d)
            if (d != split)
              st_async_f32x2(dsmem_addr(mine, static_cast<uint32_t>(d)), m_cta, l_cta,
                             dsmem_addr(bar, static_cast<uint32_t>(d)));
          s_mltab[(split * kBlockM + row) * 2 + 0] = m_cta;     // own pair
          s_mltab[(split * kBlockM + row) * 2 + 1] = l_cta;
        }
      }
      if (row == 0) WE_TRACE(232 + wg);
      if (p.nsplit == 1) {
        // no peers: normalise and store this thread's half row directly
        const float wa = w_g0 * wgt, wb = w_g1 * wgt;
#pragma unroll 1
        for (int c = 0; c < kHalf / 32; ++c) {
          uint32_t oa[32], ob[32];
          tmem_ld32(o0_addr + c * 32, oa);
          tmem_ld32(o1_addr + c * 32, ob);
          tmem_ld_wait();
          if (in_range) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float f[8];
#pragma unroll
              for (int k = 0; k < 8; ++k)
                f[k] = merge2(__uint_as_float(oa[8 * e + k]), wa, __uint_as_float(ob[8 * e + k]), wb);
              uint4 v;
              v.x = pack2<BF16>(f[0], f[1]);
              v.y = pack2<BF16>(f[2], f[3]);
              v.z = pack2<BF16>(f[4], f[5]);
              v.w = pack2<BF16>(f[6], f[7]);
              *reinterpret_cast<uint4*>(orow + c * 64 + e * 16) = v;
            }
          }
        }
      } else {
        // This split's rows, relative to its own maximum m_cta and not yet normalised, staged in the (idle) K ring
        // as fp16: every half row is divided by its largest magnitude first, so the values lie in [-1, 1] whatever
        // the range of V, and the rounding error (2^-12 of that magnitude) is far below the 2^-9 of the output's
        // own rounding.  Half as many bytes cross between the SMs as with fp32 rows.
        uint8_t* part = sK;
        const float wa = w_g0, wb = w_g1;
        float f[kHalf];
#pragma unroll
        for (int c = 0; c < kHalf / 32; ++c) {
          uint32_t oa[32], ob[32];
          if (n > 0) {
            tmem_ld32(o0_addr + c * 32, oa);
            tmem_ld32(o1_addr + c * 32, ob);
            tmem_ld_wait();
          }
          if (n > 0 && wa != 0.f && wb != 0.f) {
            // both streams contribute (the usual case): packed pairs, two instructions per pair
            const uint64_t wa2 = splat2(wa), wb2 = splat2(wb);
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const uint64_t t = fma2(pk64(oa[2 * e], oa[2 * e + 1]), wa2, fma2(pk64(ob[2 * e], ob[2 * e + 1]), wb2, 0ull));
              uint32_t x, y;
              upk64(t, x, y);
              f[c * 32 + 2 * e] = __uint_as_float(x);
              f[c * 32 + 2 * e + 1] = __uint_as_float(y);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              f[c * 32 + e] = n > 0 ? merge2(__uint_as_float(oa[e]), wa, __uint_as_float(ob[e]), wb) : 0.f;
          }
        }
        float am4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int e = 0; e < kHalf; e += 8) {
          am4[0] = max3(am4[0], fabsf(f[e + 0]), fabsf(f[e + 1]));
          am4[1] = max3(am4[1], fabsf(f[e + 2]), fabsf(f[e + 3]));
          am4[2] = max3(am4[2], fabsf(f[e + 4]), fabsf(f[e + 5]));
          am4[3] = max3(am4[3], fabsf(f[e + 6]), fabsf(f[e + 7]));
        }
        const float amax = fmaxf(fmaxf(am4[0], am4[1]), fmaxf(am4[2], am4[3]));
        const float ainv = amax > 0.f ? __fdividef(1.0f, amax) : 0.f;
        uint8_t* prow = part + row * Cfg::kPartRowB;
#pragma unroll
        for (int e = 0; e < kHalf / 8; ++e) {
          uint4 v;
          v.x = pack2<false>(f[8 * e + 0] * ainv, f[8 * e + 1] * ainv);
          v.y = pack2<false>(f[8 * e + 2] * ainv, f[8 * e + 3] * ainv);
          v.z = pack2<false>(f[8 * e + 4] * ainv, f[8 * e + 5] * ainv);
          v.w = pack2<false>(f[8 * e + 6] * ainv, f[8 * e + 7] * ainv);
          *reinterpret_cast<uint4*>(prow + wg * kHalf * 2 + e * 16) = v;
        }
        *reinterpret_cast<float*>(prow + DH * 2 + 4 * wg) = amax;
        fence_proxy_async_smem();        // the rows are read by bulk copies (async proxy) below
      }
      if (row == 0) WE_TRACE(234 + wg);
    } else {
      // ------------------------------- workspace path: hand the CTA's partial over through global memory
      float acc[kHalf];
#pragma unroll
      for (int c = 0; c < kHalf / 32; ++c) {
        uint32_t oa[32], ob[32];
        if (n > 0) {
          tmem_ld32(o0_addr + c * 32, oa);
          tmem_ld32(o1_addr + c * 32, ob);
          tmem_ld_wait();
        }
#pragma unroll
        for (int e = 0; e < 32; ++e)
          acc[c * 32 + e] = n > 0 ? merge2(__uint_as_float(oa[e]), w_g0, __uint_as_float(ob[e]), w_g1) : 0.f;
      }
      const int unit = (b * p.Hq + h) * p.n_qtiles + qt;
      // Partial result of this split, column-major so that the 128 row-threads store coalesced.
      float* wo = p.ws_o + (static_cast<int64_t>(unit) * p.nsplit + split) * (DH * kBlockM);
      float* wml = p.ws_ml + (static_cast<int64_t>(unit) * p.nsplit + split) * (2 * kBlockM);
#pragma unroll
      for (int e = 0; e < kHalf; ++e) __stcg(wo + (col0 + e) * kBlockM + row, acc[e]);
      if (wg == 0) {
        __stcg(wml + row, m_cta);
        __stcg(wml + kBlockM + row, l_cta);
      }
      __threadfence();
      named_bar_sync(1, kSoftmaxThreads);
      if (tid == 0) *s_ticket = static_cast<uint32_t>(atomicAdd(p.ws_cnt + unit, 1));
      named_bar_sync(1, kSoftmaxThreads);
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
#pragma unroll
        for (int e = 0; e < kHalf; ++e) acc[e] = 0.f;
        float den = 0.f;
        for (int s2 = 0; s2 < p.nsplit; ++s2) {
          const float ls = __ldcg(ml0 + s2 * 2 * kBlockM + kBlockM + row);
          const float ms = __ldcg(ml0 + s2 * 2 * kBlockM + row);
          if (!(ls > 0.f)) continue;
          const float w2 = fast_exp2(ms - m_all);
          den += ls * w2;
          const float* os2 = o0 + static_cast<int64_t>(s2) * (DH * kBlockM) + col0 * kBlockM + row;
#pragma unroll
          for (int e = 0; e < kHalf; ++e) acc[e] = fmaf(w2, __ldcg(os2 + e * kBlockM), acc[e]);
        }
        const float inv = (1.0f / den) * row_gate(row);
        if (in_range) {
#pragma unroll
          for (int e = 0; e < kHalf / 8; ++e) {
            uint4 v;
            v.x = pack2<BF16>(acc[8 * e + 0] * inv, acc[8 * e + 1] * inv);
            v.y = pack2<BF16>(acc[8 * e + 2] * inv, acc[8 * e + 3] * inv);
            v.z = pack2<BF16>(acc[8 * e + 4] * inv, acc[8 * e + 5] * inv);
            v.w = pack2<BF16>(acc[8 * e + 6] * inv, acc[8 * e + 7] * inv);
            *reinterpret_cast<uint4*>(orow + e * 16) = v;
          }
        }
      }
    }
  } else {
    // warp 11: with the fused append on an unfrozen write step, one CTA per batch row marks the ring slot as
    // written (LayerKVCache.upsert, src/model/kv_cache.py:151); the rows themselves are persisted by the
    // K producers of the CTAs that work for the kv head, a job or two each.
    if (p.fused && !p.is_frozen && hide_i && h == 0 && qt == 0 && split == 0) {
      uint8_t* w = p.written_w + b * p.written_batch_stride + slot_base;
      for (int t = lane; t < p.T; t += 32) w[t] = 1;
    }
    // ... and its first lane issues the tensor products of the odd tiles
    if (lane == 0 && n > 1) issue_products(1);
    __syncwarp();
  }

  // ------------------------------------------------ merge of the splits through cluster shared memory
  // CTA `split` of the cluster produces rows [r0, r1) of the query tile.  Every CTA pushes, with one bulk
  // copy per peer, the rows that peer owns (un-normalised, relative to this split's maximum) into the peer's
  // receive buffer (the idle V ring); the owner weights and adds its own rows and the received ones in split
  // order, so reruns are bit-identical.
  if (p.cluster_merge && p.nsplit > 1 && warp < 8) {
    // Only the 256 threads that staged the rows take part: a barrier among them, not the whole CTA.
    // Compiled once per split count, so that every division is by a constant and no loop carries dead iterations.
    auto merge_splits = [&](auto ns_const) {
      constexpr int NS = decltype(ns_const)::value;
      constexpr int R = kBlockM / NS;                     // rows this CTA owns
      constexpr int kRowB = Cfg::kPartRowB;
      constexpr int kTpr = 2 * NS;                        // threads per owned row in the sum (256 / R)
      constexpr int kGroups = DH / 8;                     // groups of 8 columns = 16 bytes of fp16
      constexpr int kIt = kGroups >= kTpr ? kGroups / kTpr : 1;
      constexpr int kGroupsPerHalf = kGroups / 2;
      const int r0 = R * split;
      uint8_t* part = sK;
      uint8_t* recv = sV;
      if (lane == 0) WE_TRACE(244 + warp);
      named_bar_sync(1, kSoftmaxThreads);           // this CTA's rows are staged
      // One courier thread per peer (lane 0 of warp `peer`) sends that peer its rows and, once this CTA's own
      // inbox is full, the acknowledgement.
      const int rl = tid / kTpr;
      const int cg0 = tid % kTpr;
      const bool courier = lane == 0 && warp < NS && warp != split;
      if (tid == 0) WE_TRACE(236);
      if (courier) {
        const int d = warp;
        // once all peers' pairs are here their main loops are over, so their V rings may be written
        WE_WAIT(ml_bar, 0);
        const int my_slot = split < d ? split : split - 1;          // my position among d's peers
        const uint32_t dst = dsmem_addr(smem_u32(recv) + static_cast<uint32_t>(my_slot * R * kRowB),
                                        static_cast<uint32_t>(d));
        const uint32_t bar = dsmem_addr(smem_u32(recv_bar), static_cast<uint32_t>(d));
        bulk_copy_to_peer(dst, smem_u32(part + d * R * kRowB), static_cast<uint32_t>(R * kRowB), bar);
      }
      // (asynchronous stores and bulk copies complete on the barrier through the async proxy, like any TMA
      // copy: the ordinary wait of the receiving CTA orders the data)
      WE_WAIT(ml_bar, 0);           // all pairs present
      if (tid == 0) WE_TRACE(242);
      // 2 NS threads share one of the R = 128 / NS rows; each takes every (2 NS)-th group of 8 columns (eight
      // neighbouring lanes read one 128-byte line: no bank conflicts).  Split u's half row enters with the weight
      // exp2(m_u - m_row) / l_row times its magnitude, l_row = sum over splits of l_u exp2(m_u - m_row).
      const int row = r0 + rl;
      float w_u[NS], l_u[NS];
      float m_all = -INFINITY;
#pragma unroll
      for (int u = 0; u < NS; ++u) {
        const float2 ml = *reinterpret_cast<const float2*>(s_mltab + (u * kBlockM + row) * 2);
        l_u[u] = ml.y;
        w_u[u] = ml.y > 0.f ? ml.x : -INFINITY;
        m_all = fmaxf(m_all, w_u[u]);
      }
      float den = 0.f;
#pragma unroll
      for (int u = 0; u < NS; ++u) {
        w_u[u] = l_u[u] > 0.f ? fast_exp2(w_u[u] - m_all) : 0.f;
        den = fmaf(l_u[u], w_u[u], den);
      }
      const float inv = (den > 0.f ? __fdividef(1.0f, den) : 0.f) * row_gate(row);
#pragma unroll
      for (int u = 0; u < NS; ++u) w_u[u] *= inv;
      if (tid == 0) WE_TRACE(239);
      WE_WAIT(recv_bar, 0);         // the rows of all peers have landed
      if (tid == 0) WE_TRACE(237);
      // acknowledge to the sender: its staging buffer is no longer read
      if (courier) mbar_arrive_remote(dsmem_addr(smem_u32(ack_bar), static_cast<uint32_t>(warp)));
      uint8_t* orow = static_cast<uint8_t*>(p.out) +
                      2 * (b * p.os[0] + h * p.os[1] + static_cast<int64_t>(q0 + row) * p.os[2]);
      const bool in_range = q0 + row < p.T;
      const bool active = cg0 < kGroups;       // (more threads than column groups only at DH = 64 with 8 splits)
      float acc[kIt][8];
#pragma unroll
      for (int k = 0; k < kIt; ++k)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[k][e] = 0.f;
#pragma unroll
      for (int u = 0; u < NS; ++u) {
        const uint8_t* src = u == split ? part + row * kRowB : recv + ((u < split ? u : u - 1) * R + rl) * kRowB;
        const float2 mag = *reinterpret_cast<const float2*>(src + DH * 2);
        const float w0 = w_u[u] * mag.x, w1 = w_u[u] * mag.y;
#pragma unroll
        for (int k = 0; k < kIt; ++k) {
          const int cg = cg0 + k * kTpr;
          if (active) {
            const float w = cg < kGroupsPerHalf ? w0 : w1;
            const uint4 v = *reinterpret_cast<const uint4*>(src + cg * 16);
            const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&vv[e]));
              acc[k][2 * e + 0] = fmaf(w, x.x, acc[k][2 * e + 0]);
              acc[k][2 * e + 1] = fmaf(w, x.y, acc[k][2 * e + 1]);
            }
          }
        }
      }
      if (tid == 0) WE_TRACE(243);
      if (in_range && active) {
#pragma unroll
        for (int k = 0; k < kIt; ++k) {
          const int cg = cg0 + k * kTpr;
          uint4 v;
          v.x = pack2<BF16>(acc[k][0], acc[k][1]);
          v.y = pack2<BF16>(acc[k][2], acc[k][3]);
          v.z = pack2<BF16>(acc[k][4], acc[k][5]);
          v.w = pack2<BF16>(acc[k][6], acc[k][7]);
          *reinterpret_cast<uint4*>(orow + cg * 16) = v;
        }
      }
    };
    if (p.nsplit == 2) merge_splits(std::integral_constant<int, 2>{});
    else if (p.nsplit == 4) merge_splits(std::integral_constant<int, 4>{});
    else merge_splits(std::integral_constant<int, 8>{});
    if (tid == 0) WE_TRACE(238);
    if (tid == kAttnThreads - 1) WE_TRACE(241);
    // This CTA may leave once every peer has acknowledged the rows pushed to it; nothing else of this CTA is
    // touched by a peer after that (their pairs and rows arrived before this CTA summed).
    WE_WAIT(ack_bar, 0);
  }

  // --------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (tid == 0) WE_TRACE(228);
  if (*s_abort != 0) {
    if (tid == 0) WE_TRACE_VAL(229, *s_abort);
#ifdef WE_ATTN_DEBUG
    if (tid == 0 && p.status != nullptr) atomicExch(p.status, WE_B200_ST_WAIT_EXPIRED | (*s_abort << 8));
#else
    if (tid == 0 && p.status != nullptr) atomicExch(p.status, WE_B200_ST_WAIT_EXPIRED);
#endif
    __nanosleep(1000000);  // let copies and MMAs that are still in flight land before the CTA goes away
    __syncthreads();
  }
  if (warp == 9) {
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
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? WE_B200_OK : WE_B200_E_DRIVER;
}

// Per-device facts are cached in atomics: several host threads may call the library at once (one per engine),
// and the worst a race can do is ask the driver twice for the same answer.
constexpr int kMaxDevices = 64;

static int sm_count() {
  static std::atomic<int> cached[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      return 148;                 // (not cached: the next call asks again)
    }
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
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
  // Split count: a power of two up to 8 (one thread-block cluster), chosen by a small cost model:
  // waves of CTAs x (key tiles per CTA + fixed per-CTA cost in tile units: prologue, epilogue, merge).
  const int sms = sm_count();
  int ns = 1;
  double best = 0.0;
  for (int cand = 1; cand <= 8 && cand <= s.ntiles; cand *= 2) {
    const long long ctas = static_cast<long long>(s.units) * cand;
    const double waves = static_cast<double>((ctas + sms - 1) / sms);
    const double tiles = static_cast<double>((s.ntiles + cand - 1) / cand);
    const double cost = waves * (tiles + (cand == 1 ? 6.0 : 10.0));
    if (cand == 1 || cost < best * 0.98) {   // a finer split must win by a margin
      best = cost;
      ns = cand;
    }
  }
  s.nsplit = ns;
  s.o_bytes = ns > 1 ? static_cast<size_t>(s.units) * ns * Dh * kBlockM * sizeof(float) : 0;
  s.ml_bytes = ns > 1 ? static_cast<size_t>(s.units) * ns * 2 * kBlockM * sizeof(float) : 0;
  s.cnt_bytes = ((static_cast<size_t>(s.units) * sizeof(int32_t)) + 255) & ~static_cast<size_t>(255);
  return s;
}

// The opt-in shared-memory size of a kernel variant is set once per device.
template <int DH, bool BF16>
static cudaError_t ensure_smem_attribute(int dev) {
  static std::atomic<bool> done[kMaxDevices];
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  if (done[dev].load(std::memory_order_acquire)) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(frame_attn_kernel<DH, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             AttnCfg<DH>::kSmemBytes);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return e;
  }
  done[dev].store(true, std::memory_order_release);
  return cudaSuccess;
}

// How many clusters of `cluster` CTAs of this kernel can be resident at once on the current device
// (cached per device and cluster size; 0 = clusters of that size cannot be launched; a failed query is
// reported as 0 but not cached).
template <int DH, bool BF16>
static int max_active_clusters(int dev, int cluster) {
  static std::atomic<int> cached[kMaxDevices][9];   // value + 1; 0 = not asked yet
  if (dev < 0 || dev >= kMaxDevices || cluster < 1 || cluster > 8) return 0;
  const int have = cached[dev][cluster].load(std::memory_order_relaxed);
  if (have != 0) return have - 1;
  if (ensure_smem_attribute<DH, BF16>(dev) != cudaSuccess) return 0;   // the query needs the opt-in size set
  using Cfg = AttnCfg<DH>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(cluster) * 64u, 1, 1);
  cfg.blockDim = dim3(kAttnThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(cluster);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, frame_attn_kernel<DH, BF16>, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  cached[dev][cluster].store(n + 1, std::memory_order_relaxed);
  return n;
}

// Can the splits of a query tile merge through cluster shared memory for this kernel variant?
// Setting the environment variable WE_B200_FORCE_WORKSPACE_MERGE to a non-empty value other than "0" answers
// "no" for every split plan: the splits then merge through the caller's workspace, the path a device takes on
// which clusters of that size cannot be scheduled.  (For testing that path on devices where they can.)
static bool cluster_merge_available(int Dh, int dtype, int nsplit) {
  if (nsplit == 1) return true;
  if (nsplit > 8) return false;
  const char* force = getenv("WE_B200_FORCE_WORKSPACE_MERGE");
  if (force != nullptr && force[0] != '\0' && !(force[0] == '0' && force[1] == '\0')) return false;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  if (Dh == 128) {
    return (dtype == WE_B200_BF16 ? max_active_clusters<128, true>(dev, nsplit)
                                  : max_active_clusters<128, false>(dev, nsplit)) >= 1;
  }
  return (dtype == WE_B200_BF16 ? max_active_clusters<64, true>(dev, nsplit)
                                : max_active_clusters<64, false>(dev, nsplit)) >= 1;
}

template <int DH, bool BF16>
static int launch_variant(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tkn,
                          const CUtensorMap& tvn, AttnParams p, dim3 grid, bool overlap_previous_kernel,
                          cudaStream_t stream) {
  using Cfg = AttnCfg<DH>;
  int dev = 0;
  cudaError_t e0 = cudaGetDevice(&dev);
  if (e0 == cudaSuccess) e0 = ensure_smem_attribute<DH, BF16>(dev);
  if (e0 != cudaSuccess) return static_cast<int>(e0);
  // p.cluster_merge was decided by the caller (cluster_merge_available)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kAttnThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n_attr = 0;
  if (p.cluster_merge) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = static_cast<unsigned>(p.nsplit);
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  (void)overlap_previous_kernel;
  {
    // Programmatic dependent launch, always: the CTAs may be scheduled while the preceding kernel of the
    // stream is still draining (if that kernel allows it; otherwise this is an ordinary launch).  The kernel
    // waits for its predecessor (griddepcontrol.wait) before its first access to global memory.
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = n_attr ? attr : nullptr;
  cfg.numAttrs = n_attr;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, frame_attn_kernel<DH, BF16>, tq, tk, tv, tkn, tvn, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (e != cudaSuccess) return static_cast<int>(e);
  const cudaError_t e2 = cudaGetLastError();
  return e2 == cudaSuccess ? WE_B200_OK : static_cast<int>(e2);
}

int frame_attn_launch(const void* q, const int64_t* qs, void* out, const int64_t* os, int Hq, const void* kv,
                      const uint8_t* written, const int64_t* frame_t, const we_b200_cache_geom* g, float scale,
                      void* workspace, size_t workspace_bytes, int32_t* status, bool after_append,
                      const FusedAppend* fa, cudaStream_t stream, const OutputGate* og) {
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
  // Splits of one query tile merge through cluster shared memory whenever a cluster of that size can be
  // scheduled at all (the CTAs of one cluster are always co-resident); only otherwise through the workspace.
  const bool cluster_ok = cluster_merge_available(g->Dh, g->dtype, sp.nsplit);
  const size_t need = sp.o_bytes + sp.ml_bytes + sp.cnt_bytes;
  if (!cluster_ok) {
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
  p.ring_frames = static_cast<int32_t>(g->L / g->T);
  p.nsplit = sp.nsplit;
  p.n_qtiles = sp.n_qtiles;
  p.log2_nsplit = sp.nsplit == 8 ? 3 : (sp.nsplit == 4 ? 2 : (sp.nsplit == 2 ? 1 : 0));
  p.gqa = Hq / g->Hkv;
  p.hid_tiles_max = g->T / kBlockN;
  p.scale_log2 = (scale > 0.f ? scale : 1.0f / sqrtf(static_cast<float>(g->Dh))) * 1.4426950408889634f;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  p.ws_cnt = reinterpret_cast<int32_t*>(ws);
  p.ws_ml = reinterpret_cast<float*>(ws + sp.cnt_bytes);
  p.ws_o = reinterpret_cast<float*>(ws + sp.cnt_bytes + sp.ml_bytes);
  p.status = status;
  CUtensorMap tq, tk, tv, tkn, tvn;
  const int64_t kvs[3] = {g->kv_batch_stride, C * g->Dh, static_cast<int64_t>(g->Dh)};
  if ((rc = make_map(&tq, q, g->dtype, g->T, Hq, g->B, g->Dh, qs, p.q_perm)) != WE_B200_OK) return rc;
  if ((rc = make_map(&tk, kv, g->dtype, C, g->Hkv, g->B, g->Dh, kvs, p.kv_perm)) != WE_B200_OK) return rc;
  int32_t perm_v[3];
  const uint8_t* v_base = static_cast<const uint8_t*>(kv) + 2 * g->kv_plane_stride;
  if ((rc = make_map(&tv, v_base, g->dtype, C, g->Hkv, g->B, g->Dh, kvs, perm_v)) != WE_B200_OK) return rc;

  p.cluster_merge = cluster_ok ? 1 : 0;
  tkn = tk;
  tvn = tv;
  p.fused = 0;
  p.is_frozen = 0;
  p.written_w = nullptr;
  p.gate = nullptr;
  p.gate_logits = 0;
  for (int i = 0; i < 3; ++i) p.gate_s[i] = 0;
  if (og != nullptr && og->gate != nullptr) {
    if (og->gs == nullptr) return WE_B200_E_NULL;
    for (int i = 0; i < 3; ++i) {
      if (og->gs[i] < 0) return WE_B200_E_SHAPE;
      p.gate_s[i] = og->gs[i];
    }
    if (reinterpret_cast<uintptr_t>(og->gate) & 1u) return WE_B200_E_ALIGN;
    p.gate = static_cast<const uint16_t*>(og->gate);
    p.gate_logits = og->is_logits ? 1 : 0;
  }
  for (int i = 0; i < 3; ++i) p.kn_perm[i] = p.vn_perm[i] = i;
  if (fa != nullptr) {
    // the append rides along: new rows are read through their own tensor maps and written back through the
    // cache's maps, so the writable cache pointer must be the buffer the maps were made for
    if (!fa->k_new || !fa->v_new || !fa->kv_w || !fa->written_w) return WE_B200_E_NULL;
    if (fa->kv_w != kv) return WE_B200_E_SHAPE;
    if ((rc = check_strides(fa->ks, 2)) != WE_B200_OK) return rc;
    if ((rc = check_strides(fa->vs, 2)) != WE_B200_OK) return rc;
    if (!aligned16(fa->k_new) || !aligned16(fa->v_new)) return WE_B200_E_ALIGN;
    if ((rc = make_map(&tkn, fa->k_new, g->dtype, g->T, g->Hkv, g->B, g->Dh, fa->ks, p.kn_perm)) != WE_B200_OK) return rc;
    if ((rc = make_map(&tvn, fa->v_new, g->dtype, g->T, g->Hkv, g->B, g->Dh, fa->vs, p.vn_perm)) != WE_B200_OK) return rc;
    p.fused = 1;
    p.is_frozen = fa->is_frozen ? 1 : 0;
    p.written_w = fa->written_w;
  }
  if (!cluster_ok && sp.nsplit > 1) {
    // The workspace keeps whatever an earlier call left in it, and a call of another shape lays its partial
    // results where this one has its arrival counters: clear the counters on the caller's stream, now that every
    // argument has been accepted and a launch will follow.
    const cudaError_t e = cudaMemsetAsync(workspace, 0, sp.cnt_bytes, stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  dim3 grid(static_cast<unsigned>(sp.n_qtiles * sp.nsplit), static_cast<unsigned>(Hq), static_cast<unsigned>(g->B));
  if (g->Dh == 128) {
    return g->dtype == WE_B200_BF16 ? launch_variant<128, true>(tq, tk, tv, tkn, tvn, p, grid, after_append, stream)
                                    : launch_variant<128, false>(tq, tk, tv, tkn, tvn, p, grid, after_append, stream);
  }
  return g->dtype == WE_B200_BF16 ? launch_variant<64, true>(tq, tk, tv, tkn, tvn, p, grid, after_append, stream)
                                  : launch_variant<64, false>(tq, tk, tv, tkn, tvn, p, grid, after_append, stream);
}

}  // namespace we

#ifdef WE_ATTN_DEBUG
// Switches the deliberate expiry of one wait on (non-zero) or off: see g_expire_test.
extern "C" __attribute__((visibility("default"))) int we_b200_debug_expire_wait(int on) {
  return static_cast<int>(cudaMemcpyToSymbol(we::g_expire_test, &on, sizeof(on)));
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
                               workspace, workspace_bytes, status, false, nullptr, static_cast<cudaStream_t>(stream));
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
// 12 MiB: enough for the split plans of the layer shapes this library is built for (B x heads x query tiles up to
// a few hundred units of 8 splits at Dh = 128).  The scratch is only touched when the splits cannot merge through
// cluster shared memory; plans that would then need more are rejected with WE_B200_E_STATIC_SCRATCH.
constexpr size_t kStaticScratchBytes = 12u << 20;
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
  static void* scratch_of_device[we::kMaxDevices] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= we::kMaxDevices) return WE_B200_E_LIMIT;
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
  if (sp.cnt_bytes > we::kStaticScratchBytes) return WE_B200_E_STATIC_SCRATCH;
  if (sp.o_bytes + sp.ml_bytes + sp.cnt_bytes > we::kStaticScratchBytes &&
      !we::cluster_merge_available(geom_host->Dh, geom_host->dtype, sp.nsplit))
    return WE_B200_E_STATIC_SCRATCH;   // the splits would have to merge through more scratch than the array holds
  // Every other argument is checked by the launcher before anything is enqueued; it also clears the arrival
  // counters at the head of the scratch when (and only when) the launch is going to use them.
  return we::frame_attn_launch(q, q_strides_host, out, out_strides_host, Hq, kv, written, frame_t, geom_host, scale,
                               scratch, we::kStaticScratchBytes, status, false, nullptr,
                               static_cast<cudaStream_t>(stream), nullptr);
}
