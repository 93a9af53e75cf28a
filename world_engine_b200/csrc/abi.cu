// C-ABI glue of libwe_b200: version, error strings, launch counter and the
// entry points that only forward to a kernel launcher.
#include "common.cuh"

namespace we {
std::atomic<uint64_t> g_launches{0};
}

extern "C" int we_b200_abi_version(void) { return WE_B200_ABI_VERSION; }

extern "C" const char* we_b200_strerror(int code) {
  switch (code) {
    case WE_B200_OK: return "ok";
    case WE_B200_E_NULL: return "a required pointer is null";
    case WE_B200_E_ALIGN: return "a pointer or stride is not 16-byte aligned";
    case WE_B200_E_SHAPE: return "inconsistent cache geometry or strides";
    case WE_B200_E_DTYPE: return "dtype or head_dim not supported by this kernel";
    case WE_B200_E_WORKSPACE: return "workspace missing or too small";
    case WE_B200_E_DRIVER: return "tensor-map encoder unavailable or rejected the layout";
    case WE_B200_E_LIMIT: return "a size exceeds a documented maximum";
    case WE_B200_E_STATIC_SCRATCH:
      return "this shape needs more split-KV scratch than the 12 MiB built into we_b200_frame_attn_static; "
             "use we_b200_frame_attn with a caller-provided workspace";
    default: break;
  }
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "unknown we_b200 error";
}

extern "C" uint64_t we_b200_launch_count(void) { return we::g_launches.load(std::memory_order_relaxed); }

extern "C" int we_b200_kv_append(const void* k_new, const int64_t* k_strides_host, const void* v_new,
                                 const int64_t* v_strides_host, void* kv, uint8_t* written, uint8_t* mask_written,
                                 const int64_t* frame_t, const we_b200_cache_geom* geom_host, int is_frozen,
                                 void* stream) {
  return we::kv_append_launch(k_new, k_strides_host, v_new, v_strides_host, kv, written, mask_written, frame_t,
                              geom_host, is_frozen, static_cast<cudaStream_t>(stream));
}

static int append_attend_impl(const void* q, const int64_t* q_strides_host, void* out,
                              const int64_t* out_strides_host, int32_t Hq, const void* k_new,
                              const int64_t* k_strides_host, const void* v_new, const int64_t* v_strides_host,
                              void* kv, uint8_t* written, uint8_t* mask_written, const int64_t* frame_t,
                              const we_b200_cache_geom* geom_host, int is_frozen, float scale,
                              const we::OutputGate* gate, void* workspace, size_t workspace_bytes, int32_t* status,
                              void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // One launch does both when the tail frame is made of whole 128-key tiles and nobody asked for the
  // visibility vector: the attention kernel reads the tiles of the new frame from k_new / v_new and stores them
  // from shared memory into the cache.  Otherwise: the append kernel, then the attention kernel (which overlaps
  // its on-chip set-up with the append through programmatic dependent launch).
  const bool two_byte = geom_host != nullptr && (geom_host->dtype == WE_B200_BF16 || geom_host->dtype == WE_B200_F16);
  if (two_byte && mask_written == nullptr && geom_host->T % 128 == 0 && geom_host->L % 128 == 0 && k_new && v_new &&
      kv && written && geom_host->Dh % 8 == 0) {
    const we::FusedAppend fa = {k_new, k_strides_host, v_new, v_strides_host, kv, written, is_frozen};
    return we::frame_attn_launch(q, q_strides_host, out, out_strides_host, Hq, kv, written, frame_t, geom_host, scale,
                                 workspace, workspace_bytes, status, /*after_append=*/false, &fa, s, gate);
  }
  const int rc = we::kv_append_launch(k_new, k_strides_host, v_new, v_strides_host, kv, written, mask_written,
                                      frame_t, geom_host, is_frozen, s);
  if (rc != WE_B200_OK) return rc;
  return we::frame_attn_launch(q, q_strides_host, out, out_strides_host, Hq, kv, written, frame_t, geom_host, scale,
                               workspace, workspace_bytes, status, /*after_append=*/true, nullptr, s, gate);
}

extern "C" int we_b200_append_attend(const void* q, const int64_t* q_strides_host, void* out,
                                     const int64_t* out_strides_host, int32_t Hq, const void* k_new,
                                     const int64_t* k_strides_host, const void* v_new, const int64_t* v_strides_host,
                                     void* kv, uint8_t* written, uint8_t* mask_written, const int64_t* frame_t,
                                     const we_b200_cache_geom* geom_host, int is_frozen, float scale, void* workspace,
                                     size_t workspace_bytes, int32_t* status, void* stream) {
  return append_attend_impl(q, q_strides_host, out, out_strides_host, Hq, k_new, k_strides_host, v_new,
                            v_strides_host, kv, written, mask_written, frame_t, geom_host, is_frozen, scale, nullptr,
                            workspace, workspace_bytes, status, stream);
}

extern "C" int we_b200_append_attend_gated(const void* q, const int64_t* q_strides_host, void* out,
                                           const int64_t* out_strides_host, int32_t Hq, const void* k_new,
                                           const int64_t* k_strides_host, const void* v_new,
                                           const int64_t* v_strides_host, void* kv, uint8_t* written,
                                           uint8_t* mask_written, const int64_t* frame_t,
                                           const we_b200_cache_geom* geom_host, int is_frozen, float scale,
                                           const void* gate, const int64_t* gate_strides_host, int gate_is_logits,
                                           void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
  if (gate == nullptr || gate_strides_host == nullptr) return WE_B200_E_NULL;
  const we::OutputGate og = {gate, gate_strides_host, gate_is_logits};
  return append_attend_impl(q, q_strides_host, out, out_strides_host, Hq, k_new, k_strides_host, v_new,
                            v_strides_host, kv, written, mask_written, frame_t, geom_host, is_frozen, scale, &og,
                            workspace, workspace_bytes, status, stream);
}
