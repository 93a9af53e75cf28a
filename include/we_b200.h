/*
 * we_b200.h -- C ABI of libwe_b200.so: frame-causal attention over the KV
 * ring-buffer cache, hand-written for NVIDIA B200 (sm_100a).
 *
 * The reference (Overworldai/world_engine) is a pure-Python PyTorch library
 * with no FFI of its own; each entry point below names the Python code whose
 * work it replaces (paths relative to the reference project root).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its name ends in `_host`.
 *   - The library owns no memory and keeps no session state: caches,
 *     `written` vectors, workspaces and status words belong to the caller.
 *   - All work is enqueued on `stream` (a cudaStream_t passed as void*);
 *     nothing synchronises with the host, so calls may be captured in a
 *     CUDA graph.  `frame_t` is read on the device for the same reason
 *     (reference: src/model/kv_cache.py:126 keeps it a device scalar).
 *   - Return value: 0 = OK; negative = argument rejected on the host before
 *     any launch (WE_B200_E_*); positive = the cudaError_t of a failed
 *     launch.  Nothing throws, aborts or traps.  Device-side anomalies (a
 *     bounded wait that expired) are written to `*status` and the kernel
 *     returns; 0 there means healthy.
 *   - Strides are in ELEMENTS.  The innermost (head_dim) axis is contiguous.
 *   - dtype codes: WE_B200_BF16, WE_B200_F16 (attention + append),
 *     WE_B200_F32 (append only).
 *
 * Cache geometry (one layer), exactly the reference's LayerKVCache
 * (src/model/kv_cache.py:70-97): ring of L tokens + one tail frame of T
 * tokens, capacity C = L + T.  Element (plane, b, h, token, d) of `kv` lives
 * at  plane*kv_plane_stride + b*kv_batch_stride + (h*C + token)*Dh + d.
 * The reference tensor kv[2,B,H,C,Dh] has kv_plane_stride = B*H*C*Dh and
 * kv_batch_stride = H*C*Dh; a slab of independent sessions [S,2,1,H,C,Dh]
 * has kv_plane_stride = H*C*Dh and kv_batch_stride = 2*H*C*Dh.
 * `written` is C bytes (0/1) per batch row, rows `written_batch_stride`
 * bytes apart (0 = one vector shared by all rows, as in the reference).
 * `frame_t` is an int64 per batch row, rows `frame_t_stride` elements apart
 * (0 = row 0's value for every row, as src/model/kv_cache.py:126 does).
 */
#ifndef WE_B200_H_
#define WE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WE_B200_ABI_VERSION 1

#if defined(__GNUC__)
#define WE_B200_API __attribute__((visibility("default")))
#else
#define WE_B200_API
#endif

enum {
  WE_B200_BF16 = 0,
  WE_B200_F16 = 1,
  WE_B200_F32 = 2
};

enum {
  WE_B200_OK = 0,
  WE_B200_E_NULL = -1,        /* a required pointer is null                     */
  WE_B200_E_ALIGN = -2,       /* a pointer or stride is not 16-byte aligned      */
  WE_B200_E_SHAPE = -3,       /* L % T != 0, T > L, dilation does not divide...  */
  WE_B200_E_DTYPE = -4,       /* dtype / head_dim unsupported by this kernel     */
  WE_B200_E_WORKSPACE = -5,   /* workspace missing or too small                  */
  WE_B200_E_DRIVER = -6,      /* tensor-map encoder unavailable / encode failed  */
  WE_B200_E_LIMIT = -7,       /* a size exceeds a documented maximum             */
  WE_B200_E_STATIC_SCRATCH = -8 /* shape needs more scratch than the built-in array of
                                   we_b200_frame_attn_static holds (12 MiB)       */
};

/* Device status codes written to *status by the attention kernel. */
enum {
  WE_B200_ST_OK = 0,
  WE_B200_ST_WAIT_EXPIRED = 1, /* a bounded mbarrier wait gave up; output invalid */
  WE_B200_ST_INDEX_RANGE = 2   /* a token position points outside the RoPE table (the row was clamped) */
};

typedef struct we_b200_cache_geom {
  int32_t B;                    /* batch rows (independent sessions)            */
  int32_t Hkv;                  /* kv heads                                      */
  int32_t T;                    /* tokens per frame                              */
  int32_t Dh;                   /* head dim                                      */
  int64_t L;                    /* ring length in tokens (multiple of T)         */
  int32_t dilation;             /* pinned_dilation, >= 1                         */
  int32_t dtype;                /* WE_B200_*                                     */
  int64_t kv_plane_stride;      /* elements between the K and the V plane        */
  int64_t kv_batch_stride;      /* elements between batch rows                   */
  int64_t written_batch_stride; /* bytes between batch rows of `written`         */
  int64_t frame_t_stride;       /* int64 elements between batch rows of frame_t  */
} we_b200_cache_geom;

/* ABI version of the loaded library (== WE_B200_ABI_VERSION of its build). */
WE_B200_API int we_b200_abi_version(void);

/* Static message for a return code of this library (or the CUDA runtime). */
WE_B200_API const char* we_b200_strerror(int code);

/*
 * Fused K/V append.  Replaces torch.stack + the two index_copy_ calls and the
 * `written` / mask bookkeeping of LayerKVCache.upsert
 * (src/model/kv_cache.py:126-151,191-193):
 *   - always copies the new frame into the tail slice [L, L+T)        (:138)
 *   - if !is_frozen and frame_t % dilation == 0, copies it into ring slot
 *     base = ((frame_t + d-1)/d % ((L/T)/d)) * T and sets written there
 *                                                              (:129-131,147-151)
 *   - if mask_written != NULL, writes the per-token visibility of this call
 *     (written with the ring slot hidden on write steps)           (:141-143)
 * k_new / v_new are [B,Hkv,T,Dh] views with strides (b,h,t) in elements.
 * One read of the new frame, 16-byte vector stores.
 */
WE_B200_API int we_b200_kv_append(const void* k_new, const int64_t* k_strides_host,
                      const void* v_new, const int64_t* v_strides_host,
                      void* kv, uint8_t* written, uint8_t* mask_written,
                      const int64_t* frame_t, const we_b200_cache_geom* geom_host,
                      int is_frozen, void* stream);

/*
 * Block-mask tables.  Replaces make_block_mask's tensor bookkeeping
 * (src/model/kv_cache.py:18-45): classifies each 128-token KV block of
 * mask_written[C] as empty / partial / full and emits flex-attention's
 * ordered form (indices of set blocks ascending, then the rest ascending --
 * what a stable descending argsort of the bool row yields).
 * Outputs are int32: *_num_blocks[q_blocks], *_indices[q_blocks*kv_blocks],
 * q_blocks = ceil(T/128), kv_blocks = ceil(C/128).
 */
WE_B200_API int we_b200_block_mask(const uint8_t* mask_written, int64_t C, int32_t T,
                       int32_t* kv_num_blocks, int32_t* kv_indices,
                       int32_t* full_kv_num_blocks, int32_t* full_kv_indices,
                       void* stream);

/*
 * Bytes of workspace we_b200_frame_attn may need for this shape on the current
 * device (split-KV partials + arrival counters).  It is only touched, and only
 * then required, when the key splits of a query tile cannot merge through
 * cluster shared memory (splits that merge that way need no workspace and the
 * pointer may be null).  Its contents need not be initialised or preserved: a
 * launch that uses it first clears its arrival counters on `stream`, so one
 * allocation serves calls of any shape it is large enough for, as long as they
 * are ordered on one stream.
 */
WE_B200_API size_t we_b200_attn_workspace_bytes(int32_t B, int32_t Hq, int32_t T, int32_t Dh, int64_t L);

/*
 * Frame-causal attention over the cache.  Replaces
 * flex_attention(q, k_full, v_full, block_mask=bm, enable_gqa=...) at
 * src/model/attn.py:116 / src/patch_model.py:133 together with the BlockMask
 * of src/model/kv_cache.py:141-144.  Must run after we_b200_kv_append of the
 * same frame on the same stream.  The T queries of the new frame attend to
 * every token with written != 0, except the ring slot this frame maps to
 * when frame_t % dilation == 0, plus the tail frame; wrap-around is index
 * arithmetic, nothing is gathered.  q / out are [B,Hq,T,Dh] views with
 * strides (b,h,t) in elements; Hq % Hkv == 0 (GQA by head broadcast).
 * scale <= 0 selects 1/sqrt(Dh).  bf16 / f16, Dh in {64, 128}.
 */
WE_B200_API int we_b200_frame_attn(const void* q, const int64_t* q_strides_host,
                       void* out, const int64_t* out_strides_host, int32_t Hq,
                       const void* kv, const uint8_t* written, const int64_t* frame_t,
                       const we_b200_cache_geom* geom_host, float scale,
                       void* workspace, size_t workspace_bytes,
                       int32_t* status, void* stream);

/*
 * we_b200_kv_append followed by we_b200_frame_attn on `stream`: one call per
 * layer-step, what Attn.forward does at src/model/attn.py:113-116.
 */
WE_B200_API int we_b200_append_attend(const void* q, const int64_t* q_strides_host,
                          void* out, const int64_t* out_strides_host, int32_t Hq,
                          const void* k_new, const int64_t* k_strides_host,
                          const void* v_new, const int64_t* v_strides_host,
                          void* kv, uint8_t* written, uint8_t* mask_written,
                          const int64_t* frame_t, const we_b200_cache_geom* geom_host,
                          int is_frozen, float scale,
                          void* workspace, size_t workspace_bytes,
                          int32_t* status, void* stream);

/*
 * we_b200_frame_attn for callers that cannot allocate device memory.  (No counterpart in the reference,
 * which lets PyTorch allocate whatever its kernels need.)  Meant for hosts that are forbidden to call
 * the device allocator while running -- a real-time frame loop that gave all GPU memory to its own arena
 * up front, a plug-in that may only use the buffers it is handed -- and therefore cannot supply the
 * split-KV workspace.  Same arguments and results as we_b200_frame_attn minus the workspace: the scratch
 * lives in a 12 MiB array inside the library image (held by every GPU that loads the library until the
 * process ends).  It is touched only when the splits of a query tile cannot merge through cluster shared
 * memory; shapes that then need more than the array holds return WE_B200_E_STATIC_SCRATCH and launch
 * nothing (we_b200_attn_workspace_bytes tells the need in advance).  The call itself performs no
 * cudaMalloc / cudaFree and calls no allocating routine; inputs, output and status word are still the
 * caller's buffers.  The first call on each device looks up the array's device address (that device
 * must be current) -- make that first call before any stream capture begins.  All calls share the one
 * array: it keeps the previous call's contents (when a launch is going to use the array, the entry
 * point first re-zeroes the small part that must start at zero, on `stream`; a call whose arguments are
 * rejected enqueues nothing), and two calls that overlap on the GPU -- different streams, or several
 * host threads -- race on it.  Keep calls to this entry point ordered on one stream per device.
 */
WE_B200_API int we_b200_frame_attn_static(const void* q, const int64_t* q_strides_host,
                              void* out, const int64_t* out_strides_host, int32_t Hq,
                              const void* kv, const uint8_t* written, const int64_t* frame_t,
                              const we_b200_cache_geom* geom_host, float scale,
                              int32_t* status, void* stream);

/*
 * we_b200_append_attend with the head gate applied to the output rows on their
 * way out (next to the hot path: src/model/attn.py:116-119, src/patch_model.py:133-137):
 *   out[b,h,t,:] = attention(...)[b,h,t,:] * g[b,h,t]
 * `gate` is a [B,Hq,T] view (strides (b,h,t) in elements) of the dtype of q;
 * with gate_is_logits != 0 the factor is sigmoid(gate) rounded to that dtype
 * (the reference's `gates = torch.sigmoid(gate_proj(x[..., :H]))`), otherwise
 * the values are used as they are.  The product is rounded once, from the fp32
 * accumulator (the reference rounds the attention output first).
 */
WE_B200_API int we_b200_append_attend_gated(const void* q, const int64_t* q_strides_host,
                                            void* out, const int64_t* out_strides_host, int32_t Hq,
                                            const void* k_new, const int64_t* k_strides_host,
                                            const void* v_new, const int64_t* v_strides_host,
                                            void* kv, uint8_t* written, uint8_t* mask_written,
                                            const int64_t* frame_t, const we_b200_cache_geom* geom_host,
                                            int is_frozen, float scale,
                                            const void* gate, const int64_t* gate_strides_host, int gate_is_logits,
                                            void* workspace, size_t workspace_bytes,
                                            int32_t* status, void* stream);

/*
 * What happens to q, k, v between the projections and the cache, in one pass
 * (next to the hot path: src/model/attn.py:105-110, src/patch_model.py:124-129):
 *   v'  = lerp(v, v1, v_lamb)                 if v1 != NULL     (torch.lerp, :105-107)
 *   q'  = rope(rms_norm(q)),  k' = rope(rms_norm(k))            (:109-110)
 * rms_norm is the weightless F.rms_norm over the head dim computed in fp32
 * (src/model/nn.py:55-56) and rounded to the tensor dtype; rope is RoPE.forward
 * (src/model/attn.py:33-40): consecutive pairs rotated in fp32 by the angles of
 * table row t*(height*width) + y*width + x (get_angles, :22-31), output laid
 * out as [first components | second components].  All tensors are [B,H,T,Dh]
 * views with strides (b,h,t) in elements, head dim contiguous; outputs may
 * alias nothing but their own input.  A position outside the table sets
 * *status to WE_B200_ST_INDEX_RANGE (the reference's index_select would raise).
 */
typedef struct we_b200_prologue_args {
  const void* q_in;  const void* k_in;  const void* v_in;
  const void* v1;                       /* value-residual source, or NULL        */
  void* q_out;  void* k_out;  void* v_out;
  int64_t q_in_strides[3], k_in_strides[3], v_in_strides[3], v1_strides[3];
  int64_t q_out_strides[3], k_out_strides[3], v_out_strides[3];
  const void* v_lamb;                   /* device scalar, dtype v_lamb_dtype      */
  int32_t v_lamb_dtype;                 /* WE_B200_BF16 / F16 / F32               */
  const float* cos_table;               /* [table_rows][Dh/2] fp32                */
  const float* sin_table;
  int64_t table_rows;
  const int64_t* t_pos;                 /* [B][T] int64, rows pos_batch_stride apart */
  const int64_t* y_pos;
  const int64_t* x_pos;
  int64_t pos_batch_stride;
  int32_t height, width;                /* latent grid of the position ids        */
  int32_t B, T, Hq, Hkv, Dh;
  int32_t dtype;                        /* WE_B200_BF16 or WE_B200_F16            */
  float eps;                            /* of the RMS norm (fp32 epsilon by default in the reference) */
} we_b200_prologue_args;

WE_B200_API int we_b200_qkv_prologue(const we_b200_prologue_args* args_host, int32_t* status, void* stream);

/* Number of kernels the previous three entry points have launched in this
 * process (diagnostic counter for benchmarks; relaxed atomics). */
WE_B200_API uint64_t we_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* WE_B200_H_ */
