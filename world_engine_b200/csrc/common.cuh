// Shared host-side helpers of libwe_b200: argument checks, launch counter,
// device attributes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/we_b200.h"

namespace we {

extern std::atomic<uint64_t> g_launches;

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int elem_bytes(int dtype) {
  switch (dtype) {
    case WE_B200_BF16:
    case WE_B200_F16: return 2;
    case WE_B200_F32: return 4;
    default: return 0;
  }
}

// Geometry checks shared by every entry point (mirrors the reference's
// eager-only torch._check block, src/model/kv_cache.py:112-124, plus what the
// vectorised kernels need).
inline int check_geom(const we_b200_cache_geom* g) {
  if (g == nullptr) return WE_B200_E_NULL;
  const int eb = elem_bytes(g->dtype);
  if (eb == 0) return WE_B200_E_DTYPE;
  if (g->B < 1 || g->Hkv < 1 || g->T < 1 || g->Dh < 1 || g->L < 1 || g->dilation < 1) return WE_B200_E_SHAPE;
  if (g->T > g->L || g->L % g->T != 0) return WE_B200_E_SHAPE;            // :115-117
  if ((g->L / g->T) % g->dilation != 0) return WE_B200_E_SHAPE;            // :78
  if ((static_cast<int64_t>(g->Dh) * eb) % 16 != 0) return WE_B200_E_ALIGN;
  if ((g->kv_plane_stride * eb) % 16 != 0 || (g->kv_batch_stride * eb) % 16 != 0) return WE_B200_E_ALIGN;
  if (g->kv_plane_stride < 0 || g->kv_batch_stride < 0 || g->written_batch_stride < 0 || g->frame_t_stride < 0)
    return WE_B200_E_SHAPE;
  return WE_B200_OK;
}

inline int check_strides(const int64_t* s, int eb) {
  if (s == nullptr) return WE_B200_E_NULL;
  for (int i = 0; i < 3; ++i) {
    if (s[i] < 0) return WE_B200_E_SHAPE;
    if ((s[i] * eb) % 16 != 0) return WE_B200_E_ALIGN;
  }
  return WE_B200_OK;
}

// Slot arithmetic of src/model/kv_cache.py:129-131,140 (frame_t >= 0).
struct SlotInfo {
  int64_t base;     // first ring token of the slot this frame maps to
  int write_step;   // frame_t % dilation == 0
};
__host__ __device__ inline SlotInfo slot_of(int64_t frame_t, int64_t L, int T, int dilation) {
  const int64_t d = dilation;
  const int64_t num_buckets = (L / T) / d;
  const int64_t bucket = (frame_t + (d - 1)) / d;
  SlotInfo s;
  s.base = (bucket % num_buckets) * T;
  s.write_step = (frame_t % d) == 0;
  return s;
}

int kv_append_launch(const void* k_new, const int64_t* ks, const void* v_new, const int64_t* vs, void* kv,
                     uint8_t* written, uint8_t* mask_written, const int64_t* frame_t, const we_b200_cache_geom* g,
                     int is_frozen, cudaStream_t stream);

// The append of the same layer-step, when it is to ride along inside the attention launch.
struct FusedAppend {
  const void* k_new;
  const int64_t* ks;   // strides (b, h, t) in elements
  const void* v_new;
  const int64_t* vs;
  void* kv_w;
  uint8_t* written_w;
  int is_frozen;
};

// A per-(batch row, head, token) factor applied to the output rows on their way out.
struct OutputGate {
  const void* gate;       // [B,H,T] view, same 16-bit dtype as q
  const int64_t* gs;      // strides (b, h, t) in elements
  int is_logits;          // 1: the factor is sigmoid(value), rounded to the dtype like the reference's tensor
};

int frame_attn_launch(const void* q, const int64_t* qs, void* out, const int64_t* os, int Hq, const void* kv,
                      const uint8_t* written, const int64_t* frame_t, const we_b200_cache_geom* g, float scale,
                      void* workspace, size_t workspace_bytes, int32_t* status, bool after_append,
                      const FusedAppend* fused_append, cudaStream_t stream, const OutputGate* gate = nullptr);

}  // namespace we
