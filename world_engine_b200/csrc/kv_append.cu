// Fused K/V append into the ring-buffer cache (sm_100a).
//
// One pass over the new frame: every 16-byte vector of k_new / v_new is read
// once and stored to the tail slice and, on an unfrozen write step, to the
// ring slot as well.  The same launch maintains `written` and (optionally)
// the per-call visibility vector.  HBM-bound byte work: coalesced 16-byte
// loads and stores, one vector per thread, the slot computed once per CTA
// from the device-resident frame counter.
//
// Semantics follow LayerKVCache.upsert, src/model/kv_cache.py:126-151.
#include "common.cuh"

namespace we {

struct AppendParams {
  const uint4* k_new;
  const uint4* v_new;
  int64_t ks[3];  // strides (b, h, t) of k_new in 16-byte vectors
  int64_t vs[3];
  uint4* kv;
  uint8_t* written;
  uint8_t* mask_written;
  const int64_t* frame_t;
  int64_t plane_stride_v;  // in 16-byte vectors
  int64_t batch_stride_v;
  int64_t written_batch_stride;
  int64_t frame_t_stride;
  int64_t L;
  int32_t B, Hkv, T, vpr;  // vpr = 16-byte vectors per (token, head) row
  int32_t dilation;
  int32_t is_frozen;
};

constexpr int kAppendThreads = 256;

__global__ void __launch_bounds__(kAppendThreads) kv_append_kernel(const AppendParams p) {
  __shared__ int64_t s_base;
  __shared__ int s_ring;  // 1 when this call also persists into the ring slot

  // Programmatic dependent launch, both ways.  This kernel may itself have been started before the kernel
  // ahead of it in the stream finished: wait for that one first (returns at once otherwise).  Only then let
  // the kernel behind it (the attention of the same layer-step) begin its prologue: that kernel may rely on
  // everything older than this append being complete, and it waits for this grid before it reads the cache.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int plane = blockIdx.y / p.B;
  const int b = blockIdx.y - plane * p.B;
  if (threadIdx.x == 0) {
    const int64_t t = p.frame_t[static_cast<int64_t>(b) * p.frame_t_stride];
    const SlotInfo s = slot_of(t, p.L, p.T, p.dilation);
    s_base = s.base;
    s_ring = (!p.is_frozen && s.write_step) ? 1 : 0;
    // bit 1: hide the slot in this call's visibility (kv_cache.py:143)
    s_ring |= s.write_step ? 2 : 0;
  }
  __syncthreads();
  const int64_t base = s_base;
  const bool to_ring = (s_ring & 1) != 0;
  const bool hide = (s_ring & 2) != 0;
  const int64_t C = p.L + p.T;

  const int64_t per_b = static_cast<int64_t>(p.Hkv) * p.T * p.vpr;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kAppendThreads + threadIdx.x;
  if (i < per_b) {
    const int v = static_cast<int>(i % p.vpr);
    const int64_t row = i / p.vpr;
    const int t = static_cast<int>(row % p.T);
    const int h = static_cast<int>(row / p.T);
    const uint4* src = plane == 0 ? p.k_new : p.v_new;
    const int64_t* st = plane == 0 ? p.ks : p.vs;
    const uint4 val = src[b * st[0] + h * st[1] + t * st[2] + v];
    uint4* dst = p.kv + plane * p.plane_stride_v + b * p.batch_stride_v + static_cast<int64_t>(h) * C * p.vpr + v;
    dst[(p.L + t) * p.vpr] = val;                                   // tail, always (kv_cache.py:138)
    if (to_ring) {
      dst[(base + t) * p.vpr] = val;                                // ring slot (kv_cache.py:149-150)
      if (plane == 0 && h == 0 && v == 0) p.written[b * p.written_batch_stride + base + t] = 1;  // :151
    }
  }

  // Visibility of this call: `written` with the slot hidden on write steps
  // (kv_cache.py:141-143).  Bytes inside the slot are forced to 0 whatever
  // `written` holds, so the concurrent update above cannot change the result.
  if (p.mask_written != nullptr && plane == 1) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kAppendThreads;
    const uint8_t* w = p.written + b * p.written_batch_stride;
    uint8_t* m = p.mask_written + b * p.written_batch_stride;
    for (int64_t j = i; j < C; j += stride) {
      const bool in_slot = hide && j >= base && j < base + p.T;
      m[j] = in_slot ? 0 : w[j];
    }
  }
}

int kv_append_launch(const void* k_new, const int64_t* ks, const void* v_new, const int64_t* vs, void* kv,
                     uint8_t* written, uint8_t* mask_written, const int64_t* frame_t, const we_b200_cache_geom* g,
                     int is_frozen, cudaStream_t stream) {
  if (!k_new || !v_new || !kv || !written || !frame_t) return WE_B200_E_NULL;
  int rc = check_geom(g);
  if (rc != WE_B200_OK) return rc;
  const int eb = elem_bytes(g->dtype);
  if ((rc = check_strides(ks, eb)) != WE_B200_OK) return rc;
  if ((rc = check_strides(vs, eb)) != WE_B200_OK) return rc;
  if (!aligned16(k_new) || !aligned16(v_new) || !aligned16(kv)) return WE_B200_E_ALIGN;
  if ((g->written_batch_stride == 0) != (g->frame_t_stride == 0)) return WE_B200_E_SHAPE;

  AppendParams p;
  const int epv = 16 / eb;  // elements per vector
  p.k_new = static_cast<const uint4*>(k_new);
  p.v_new = static_cast<const uint4*>(v_new);
  for (int i = 0; i < 3; ++i) {
    p.ks[i] = ks[i] / epv;
    p.vs[i] = vs[i] / epv;
  }
  p.kv = static_cast<uint4*>(kv);
  p.written = written;
  p.mask_written = mask_written;
  p.frame_t = frame_t;
  p.plane_stride_v = g->kv_plane_stride / epv;
  p.batch_stride_v = g->kv_batch_stride / epv;
  p.written_batch_stride = g->written_batch_stride;
  p.frame_t_stride = g->frame_t_stride;
  p.L = g->L;
  p.B = g->B;
  p.Hkv = g->Hkv;
  p.T = g->T;
  p.vpr = g->Dh / epv;
  p.dilation = g->dilation;
  p.is_frozen = is_frozen ? 1 : 0;

  const int64_t per_b = static_cast<int64_t>(p.Hkv) * p.T * p.vpr;
  const int64_t gx = (per_b + kAppendThreads - 1) / kAppendThreads;
  if (gx > 0x7FFFFFFF || 2 * static_cast<int64_t>(g->B) > 65535) return WE_B200_E_LIMIT;
  dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(2 * g->B));
  // Launched with programmatic stream serialization: its CTAs may be scheduled while the previous kernel of
  // the stream drains (they wait for it first thing), which hides the launch latency between layer-steps.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kAppendThreads, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kv_append_kernel, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (e != cudaSuccess) return static_cast<int>(e);
  const cudaError_t e2 = cudaGetLastError();
  return e2 == cudaSuccess ? WE_B200_OK : static_cast<int>(e2);
}

}  // namespace we
