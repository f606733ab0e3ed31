/*
 * libmoc_b200 - C ABI of the B200 (sm_100a) implementation of the Mixture-of-Channels sparse
 * SwiGLU FFN path.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless said otherwise; the library allocates nothing,
 *     keeps no reference to caller memory and launches on the stream it is given
 *     (a cudaStream_t passed as void*; NULL = the legacy default stream).
 *   - Functions return 0 on success or a negative MOC_ERR_* code, never throw and never
 *     exit; moc_last_error() gives the text of the calling thread's last failure.
 *   - dtype: MOC_BF16 (tensor-core path, tcgen05) or MOC_F32 (CUDA-core path). All tensors
 *     of one call share the dtype; indices are int16, masks uint32, ranks uint16.
 *   - Matrices are row-major and contiguous unless a leading dimension is given.
 *   - "tokens" = rows of the flattened activation x[tokens, d]; d = hidden size,
 *     d_ffn = intermediate size (F), k = selected channels per token.
 *
 * Each entry point names the reference interface it replaces (path:line inside
 * xiaohuangji/MoC).
 */
#ifndef MOC_B200_H_
#define MOC_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOC_B200_ABI_VERSION 1

#define MOC_BF16 0
#define MOC_F32 1

#define MOC_OK 0
#define MOC_ERR_INVALID_ARG (-1)
#define MOC_ERR_UNSUPPORTED (-2)
#define MOC_ERR_WORKSPACE (-3)
#define MOC_ERR_CUDA (-4)
#define MOC_ERR_TENSOR_MAP (-5)
#define MOC_ERR_DEVICE_TIMEOUT (-6)

/* channel selection rule */
#define MOC_SELECT_TOPK 0   /* global row-wise Top-K on the pre-SiLU gate (moc/ffn.py:144) */
#define MOC_SELECT_2OF8 1   /* top-2 of every 8 consecutive channels (moc/ffn.py:68-108) */
#define MOC_SELECT_POST_SILU_ABS 2   /* row-wise Top-K on |SiLU(gate)| (moc/ffn.py:313-369) */

int moc_b200_abi_version(void);

/* Text of the last error raised on the calling host thread ("" if none). */
const char* moc_last_error(void);

/* Layout helpers: leading dimension (elements) of dense [tokens, d_ffn] scratch rows,
 * 32-bit mask words per token, and K' of the 2:8 rule (moc/ffn.py:62-65). */
int64_t moc_ffn_ld(int64_t d_ffn);
int64_t moc_mask_words(int64_t d_ffn);
int64_t moc_select_2of8_k(int64_t d_ffn);

/* Workspace sizes in bytes for moc_ffn_fwd / moc_ffn_bwd (256-byte aligned base).
 * moc_ffn_fwd_workspace_bytes covers MOC_SELECT_TOPK and MOC_SELECT_2OF8 (two dense scratch matrices);
 * MOC_SELECT_POST_SILU_ABS keeps the score matrix as a third one: moc_ffn_fwd_workspace_bytes_select. */
int64_t moc_ffn_fwd_workspace_bytes(int dtype, int64_t tokens, int64_t d_ffn);
int64_t moc_ffn_fwd_workspace_bytes_select(int dtype, int select, int64_t tokens, int64_t d_ffn);
int64_t moc_ffn_bwd_workspace_bytes(int dtype, int64_t tokens, int64_t d_ffn);

/* out[cols, rows] = in[rows, cols]^T. Used to keep W_down^T [d_ffn, d] next to the
 * parameter W_down [d, d_ffn]; replaces `down_proj.weight.t().contiguous()`
 * (moc/inference/inference_ffn.py:104-110). */
int moc_transpose(int dtype, const void* in, void* out, int64_t rows, int64_t cols, void* stream);

/* Row-wise Top-K channel selection on a gate matrix g[tokens, ldg] (first d_ffn columns).
 * Outputs, per token: idx[k] selected channels in ascending order, g_sel[k] their gate
 * values, bitmap[moc_mask_words] selection mask, rank0[moc_mask_words] rank of each mask
 * word's first channel. Ties at the K-th value go to the lower channel index; values are
 * ordered by the IEEE total order. Replaces torch.topk(g, k, dim=-1, sorted=False) +
 * _pack_topk_idx (moc/ffn.py:144-147, :27-41) and cub_topk_idx_i32_bf16_kernel
 * (moc/inference/cuda/optimized_global_moc_ext.cu:85-125). d_ffn <= 32768. */
int moc_topk_select(int dtype, const void* g, int64_t ldg, int64_t tokens, int64_t d_ffn, int64_t k,
                    int16_t* idx, void* g_sel, uint32_t* bitmap, uint16_t* rank0, void* stream);

/* Structured selection, k = moc_select_2of8_k(d_ffn). Replaces _select_moc_2_8
 * (moc/ffn.py:68-108) and the in-kernel top-2 of
 * moc/inference/triton_fused_ffn_kernels.py:95-114. */
int moc_select_2of8(int dtype, const void* g, int64_t ldg, int64_t tokens, int64_t d_ffn, int16_t* idx,
                    void* g_sel, uint32_t* bitmap, uint16_t* rank0, void* stream);

/* C[m, n] = A[m, k] * B[n, k]^T with fp32 accumulation. a_mn / b_mn = 1 when the operand is
 * stored [k][m] / [k][n] (M or N contiguous) instead of [m][k] / [n][k]. c_transposed = 1
 * stores C^T (C[j * ldc + i]). impl: 0 = default core of the dtype (bf16: tcgen05 / TMEM,
 * CTA-pair kernel when m > 128, else the single-CTA kernel; f32: CUDA cores), 1 = CUDA-core
 * core for either dtype, 2 / 3 = force the CTA-pair / single-CTA tensor-core kernel (bf16). status: one device int, zeroed by
 * the caller, receives a code if a bounded device-side wait gives up. Stands in for the
 * `@` / nn.Linear calls of moc/ffn.py:141-163, :203-254. */
int moc_gemm(int dtype, int impl, int64_t m, int64_t n, int64_t k, const void* a, int64_t lda, int a_mn,
             const void* b, int64_t ldb, int b_mn, void* c, int64_t ldc, int c_transposed, int* status,
             void* stream);

/* MoC FFN forward: y = (mask(SiLU(x Wg^T)) * (x Wu^T)) Wd^T with the mask chosen by
 * `select`. Replaces _MoCFunction.forward / _MoCGCPFunction.forward / _MoC28Function.forward
 * (moc/ffn.py:130-173, :378-421, :266-308) including sparse_forward_aux
 * (moc/training/triton_sparse_aux.py:197-231).
 *   in : x[tokens, d], w_gate[d_ffn, d], w_up[d_ffn, d], w_down_t[d_ffn, d] (= W_down^T)
 *   out: y[tokens, d]; the saved activation set idx[tokens, k], g_sel, u_sel [tokens, k],
 *        optional s_sel, z_sel [tokens, k] (pass NULL for moc_gcp), bitmap / rank0
 *        [tokens, moc_mask_words(d_ffn)].
 * The dense G / Z' scratch lives in `workspace`; its first 256 bytes are a status area. */
int moc_ffn_fwd(int dtype, int select, int64_t tokens, int64_t d, int64_t d_ffn, int64_t k, const void* x,
                const void* w_gate, const void* w_up, const void* w_down_t, void* y, int16_t* idx, void* g_sel,
                void* u_sel, void* s_sel, void* z_sel, uint32_t* bitmap, uint16_t* rank0, void* workspace,
                int64_t workspace_bytes, void* stream);

/* MoC FFN backward. Replaces _MoCFunction.backward / _MoCGCPFunction.backward
 * (moc/ffn.py:176-259, :424-497) including scatter_sparse_to_dense and sparse_backward_aux
 * (moc/training/triton_sparse_aux.py:266-423). idx, g_sel, u_sel [tokens, k] are the forward
 * pass's outputs (the compact saved set, moc/ffn.py:166-169, :417). z_sel NULL = recompute it
 * from g_sel, u_sel (moc_gcp, moc/ffn.py:435-436); s_sel is accepted for symmetry and not read
 * (s = SiLU(g_sel) is rebuilt with the same bits). Outputs are overwritten, not accumulated: grad_x[tokens, d],
 * grad_w_gate[d_ffn, d], grad_w_up[d_ffn, d], grad_w_down[d, d_ffn] (parameter layout).
 * ev_down / ev_gate / ev_up: optional cudaEvent_t handles recorded on `stream` as soon as the
 * respective weight gradient is final, so a caller can start its all-reduce while the rest of
 * the backward pass runs. */
int moc_ffn_bwd(int dtype, int64_t tokens, int64_t d, int64_t d_ffn, int64_t k, const void* grad_y, const void* x,
                const void* w_gate, const void* w_up, const void* w_down_t, const int16_t* idx,
                const void* g_sel, const void* u_sel, const void* s_sel, const void* z_sel,
                void* grad_x, void* grad_w_gate, void* grad_w_up, void* grad_w_down, void* workspace,
                int64_t workspace_bytes, void* ev_down, void* ev_gate, void* ev_up, void* stream);

/* Dense SwiGLU FFN forward y = (SiLU(x Wg^T) * (x Wu^T)) Wd^T on the same GEMM core, the comparison
 * row of the reference (StandardSwiGLUFFN.forward, moc/ffn.py:111-121: three nn.Linear calls).
 * g_out, u_out [tokens, moc_ffn_ld(d_ffn)] receive the rounded gate / up activations, which the
 * backward pass needs (what autograd saves for the reference). Workspace as for moc_ffn_fwd. */
int moc_dense_ffn_fwd(int dtype, int64_t tokens, int64_t d, int64_t d_ffn, const void* x, const void* w_gate,
                      const void* w_up, const void* w_down_t, void* y, void* g_out, void* u_out, void* workspace,
                      int64_t workspace_bytes, void* stream);

/* Dense SwiGLU FFN backward (PyTorch autograd of moc/ffn.py:120-121). g, u: the forward pass's outputs.
 * Gradients are overwritten; grad_w_down has the parameter layout [d, d_ffn]. Workspace as for moc_ffn_bwd. */
int moc_dense_ffn_bwd(int dtype, int64_t tokens, int64_t d, int64_t d_ffn, const void* grad_y, const void* x,
                      const void* w_gate, const void* w_up, const void* w_down_t, const void* g, const void* u,
                      void* grad_x, void* grad_w_gate, void* grad_w_up, void* grad_w_down, void* workspace,
                      int64_t workspace_bytes, void* stream);

/* ---- decode path: a few token rows at a time, bf16 only (like the reference's fast paths,
 * moc/inference/cuda/optimized_global_moc_ext.cpp:67-74). x[batch, d], w_gate / w_up [d_ffn, d],
 * w_down_t[d_ffn, d] = W_down^T (the reference keeps the same copy, inference_ffn.py:104-110),
 * y[batch, d]. d % 8 == 0. All scratch (gate scores, indices, sparse z, split-K partial sums) lives in
 * `workspace` (moc_decode_workspace_bytes, 256-byte aligned); nothing is allocated. The launches are
 * stream-ordered and capturable in a CUDA graph. Results are deterministic (no floating-point
 * atomics). Batches of up to 8 rows (d a multiple of 256 up to 2048, at most 48 channels per SM, weights
 * 16-byte aligned) run as ONE persistent launch of SM-count CTAs, preceded by a small kernel that clears the
 * status area: every CTA streams the W_gate, W_up and W_down^T rows of its own channels once through a
 * shared-memory ring, and the CTAs synchronise through counters in the workspace (bounded waits;
 * moc_read_status reports a time-out): the device must be able to hold that grid at once, i.e. not be running
 * another kernel that keeps SMs busy indefinitely. Other shapes and batches of 9 to 15 rows use separate
 * streaming kernels per projection; batches of 16 rows and more (dense: 8) that the persistent launch does
 * not take run the projections on the tensor cores. ---- */
int64_t moc_decode_workspace_bytes(int64_t batch, int64_t d, int64_t d_ffn);

/* Global MoC decode FFN: gate projection, row-wise Top-K (lowest index wins ties), SiLU(g) * (x . W_up
 * rows of the selected channels), gathered down projection. Replaces
 * InferenceMoCSwiGLUFFN.moc_inference_optimized_global_after_gate_native (inference_ffn.py:182-196:
 * gate_proj + moc_native::optimized_global_after_gate_bf16) and equals masked_reference
 * (inference_ffn.py:169-180) up to bf16 rounding. */
int moc_decode_global(int64_t batch, int64_t d, int64_t d_ffn, int64_t k, const void* x, const void* w_gate,
                      const void* w_up, const void* w_down_t, void* y, void* workspace, int64_t workspace_bytes,
                      void* stream);

/* Same with the gate scores supplied by the caller (gate_scores[batch, d_ffn], contiguous): the exact
 * counterpart of moc_native::optimized_global_after_gate_bf16(x, gate_scores, up_weight, down_weight_t, k)
 * (optimized_global_moc_ext.cpp:61-76, .cu:457-540). */
int moc_decode_after_gate(int64_t batch, int64_t d, int64_t d_ffn, int64_t k, const void* x, const void* gate_scores,
                          const void* w_up, const void* w_down_t, void* y, void* workspace, int64_t workspace_bytes,
                          void* stream);

/* MoC 2:8 decode FFN: top-2 of every 8 consecutive gate channels (tail group: top-min(2, tail)), selection on
 * the bf16-rounded gate. Replaces moc::fused_grouped_top2_up_silu + moc::selected_grouped_down
 * (moc/inference/triton_grouped_moc_ops.py:26-131, triton_fused_ffn_kernels.py:30-156, :229-267); unlike
 * them it accepts d_ffn % 8 != 0. */
int moc_decode_2of8(int64_t batch, int64_t d, int64_t d_ffn, const void* x, const void* w_gate, const void* w_up,
                    const void* w_down_t, void* y, void* workspace, int64_t workspace_bytes, void* stream);

/* Dense SwiGLU decode FFN (InferenceMoCSwiGLUFFN.dense_baseline, inference_ffn.py:164-167). */
int moc_decode_dense(int64_t batch, int64_t d, int64_t d_ffn, const void* x, const void* w_gate, const void* w_up,
                     const void* w_down_t, void* y, void* workspace, int64_t workspace_bytes, void* stream);

/* sparse_z[b, k] = round(round(SiLU(g_sel[b, k])) * round(x[b, :] . w_up[idx[b, k], :])): the up projection of the
 * selected channels alone (moc_native::optimized_global_selected_up_silu_bf16,
 * optimized_global_moc_ext.cu:127-245), with int16 indices. bf16. */
int moc_decode_selected_up(int64_t batch, int64_t k, int64_t d, int64_t d_ffn, const void* x, const void* g_sel,
                           const int16_t* idx, const void* w_up, void* sparse_z, void* stream);

/* y[b, :] = sum_k sparse_z[b, k] * w_down_t[idx[b, k], :]: the gathered down projection alone
 * (moc_native::optimized_global_selected_down_bf16, optimized_global_moc_ext.cu:247-372, and
 * moc::selected_grouped_down, triton_grouped_moc_ops.py:96-131), with int16 indices. */
int moc_decode_selected_down(int64_t batch, int64_t k, int64_t d, int64_t d_ffn, const void* sparse_z,
                             const int16_t* idx, const void* w_down_t, void* y, void* workspace,
                             int64_t workspace_bytes, void* stream);

/* Global MoC decode FFN without any caller-provided scratch: same computation and same result as
 * moc_decode_global, for callers that must not allocate device memory when they call (a fixed memory
 * budget that is already handed out, a frozen allocator in a serving loop, a runtime that passes a
 * plugin nothing but its inputs and outputs). The scratch is a fixed 12 MiB array inside the library's
 * device image, present on every GPU that loads the library for the life of the process. No counterpart
 * in the reference (its decode ops allocate their outputs and temporaries with torch::empty,
 * moc/inference/cuda/optimized_global_moc_ext.cu:468-472).
 *   Limits: batch <= moc_decode_static_max_batch() (8), d <= moc_decode_static_max_d() (4096),
 *   d_ffn <= moc_decode_static_max_d_ffn() (8192); larger sizes return MOC_ERR_UNSUPPORTED.
 *   The first call on each device looks up the scratch address (the device must be current); make that
 *   first call outside any stream capture. The call itself allocates nothing.
 *   All calls on a device share the one scratch array: calls that may overlap on the GPU (different
 *   streams, or several host threads) race with each other; serialise them. Nothing in the scratch
 *   needs clearing between calls: every part is rewritten before it is read. */
int moc_decode_global_static(int64_t batch, int64_t d, int64_t d_ffn, int64_t k, const void* x, const void* w_gate,
                             const void* w_up, const void* w_down_t, void* y, void* stream);
int64_t moc_decode_static_max_batch(void);
int64_t moc_decode_static_max_d(void);
int64_t moc_decode_static_max_d_ffn(void);

/* ---- host model: the non-FFN part of one static-cache decode step (bf16) -------------------------------------
 * The reference's end-to-end decode benchmark (benchmarks/inference/benchmark_decode.py:312-362,
 * DecoderModel.forward_step_static over the blocks of moc/model.py:19-88) leaves these to chains of small PyTorch
 * operations; around a 22 us FFN they dominate the time of a token. Three launches per layer replace them. `pos`
 * is a DEVICE pointer to the int64 position of the new token, so that a captured step can be replayed.
 *
 * moc_host_rmsnorm: h [rows, d] += delta (delta may be NULL: no update), then y = RMSNorm(h) * weight with the
 *   statistics in fp32 (moc/model.py:19-27); h is updated in place. d % 8 == 0.
 * moc_host_rope_cache: qkv [batch, 3, heads, head_dim] (one row of the fused projection per batch row);
 *   q_out [batch, heads, head_dim] = rotary(q), cache_k[b, h, pos] = rotary(k), cache_v[b, h, pos] = v
 *   (moc/model.py:37-43 on interleaved pairs; caches [batch, heads, t_max, head_dim];
 *   cos_table, sin_table [t_max, head_dim / 2] bf16).
 * moc_host_attn_step: y [batch, heads * head_dim] = softmax(q . K[0..pos] / sqrt(head_dim)) V[0..pos], fp32
 *   accumulation (benchmark_decode.py:347-356). head_dim in {8, 16, 32, 64, 128}, t_max <= 11000. */
int moc_host_rmsnorm(int64_t rows, int64_t d, void* h, const void* delta, const void* weight, void* y, float eps,
                     void* stream);
int moc_host_rope_cache(int64_t batch, int64_t heads, int64_t head_dim, int64_t t_max, const void* qkv,
                        const void* cos_table, const void* sin_table, const int64_t* pos, void* q_out, void* cache_k,
                        void* cache_v, void* stream);
int moc_host_attn_step(int64_t batch, int64_t heads, int64_t head_dim, int64_t t_max, const void* q, const void* cache_k,
                       const void* cache_v, const int64_t* pos, void* y, void* stream);

/* Per-kernel timing without a profiler. Between moc_profile_begin and moc_profile_end (process-wide,
 * one profile at a time) the library records events[0], events[1], ... (a HOST array of created
 * cudaEvent_t handles, timing enabled) on the stream of each call, one right before every
 * kernel it launches and one when an FFN entry point returns. moc_profile_end copies the
 * kernel-kind tag of each recorded event to tags_out and returns their number; the time
 * between events i and i+1 is the duration of kernel i. Tags: 0 end of call, 1 tcgen05 GEMM,
 * 2 CUDA-core GEMM, 3 Top-K select, 4 2:8 select, 5 expand, 6 transpose, 7-11 decode kernels,
 * 12 sparse backward.
 * No counterpart in the reference, which times whole passes with CUDA events
 * (benchmarks/training/benchmark_training_latency.py:59-106). */
int moc_profile_begin(void** events, int capacity);
int moc_profile_end(int* tags_out, int capacity);
/* Number of GEMM launches this process has put on the library's side stream so far (the rows of a
 * product that do not fill half a 256-row tile pair run there beside the main launch); these carry
 * no profile event. No counterpart in the reference. */
int64_t moc_side_launch_count(void);
/* Data-parallel training: the dX GEMM, the last kernel of moc_ffn_bwd, leaves `sms` SMs (0..64, default 0) free
 * so that a gradient all-reduce started behind the weight-gradient events of moc_ffn_bwd runs beside it.
 * Process-wide. No counterpart in the reference (it has no distributed code). */
int moc_set_overlap_sm_reserve(int sms);

/* Data-parallel training: in-place sum (average != 0: mean) over `world` ranks (<= 8, one process per GPU of one
 * node) of a gradient buffer that every rank holds in a symmetric allocation mapped by its peers. The
 * north star asks for the weight gradients to be all-reduced over NVLink; the reference itself has no distributed
 * code, so this entry point has no counterpart there.
 *   peer_buffers[r], peer_flags[r] (HOST arrays of `world` device pointers): rank r's buffer and flag words as
 *   mapped in this process; entry `rank` is the local one. Flags: moc_symm_allreduce_flag_bytes() bytes per rank,
 *   zeroed once when the allocation is made, never touched by the caller afterwards.
 *   multicast_buffer: multicast address of the buffer (NVSwitch; the kernel then reduces in the switch with
 *   multimem.ld_reduce / multimem.st), or NULL: plain peer loads and stores.
 *   bytes: size of the buffer, a multiple of 16. call: 1, 2, 3, ... - the same sequence on every rank.
 *   ctas: CTAs of 512 threads to launch (a few per SM that the caller wants the reduction to occupy).
 * Every rank must make the same sequence of calls. Rank r reduces the r-th slice of the buffer and writes it to
 * all ranks; ranks meet before the first read and after the last write, with bounded waits (about one second):
 * after a time-out the buffer's contents are unspecified and moc_symm_allreduce_status reports
 * MOC_ERR_DEVICE_TIMEOUT. The library allocates nothing and knows nothing about how the mapping was made. */
int moc_symm_allreduce(int dtype, int rank, int world, void* const* peer_buffers, void* multicast_buffer,
                       void* const* peer_flags, int64_t bytes, int average, uint32_t call, int ctas, void* stream);
int64_t moc_symm_allreduce_flag_bytes(void);
/* Synchronises `stream`, then MOC_OK or MOC_ERR_DEVICE_TIMEOUT for the local flag words `flags`. */
int moc_symm_allreduce_status(const void* flags, void* stream);

/* Synchronises `stream` and returns MOC_OK, or MOC_ERR_DEVICE_TIMEOUT if a kernel of the
 * last call that used `workspace` recorded a bounded-wait failure in its status area. */
int moc_read_status(const void* workspace, void* stream);

/* Test hook: limit, in SM clock cycles, of the bounded grid-barrier waits of the persistent decode kernel
 * (copy-completion waits keep their fixed limit, so that no CTA leaves with a copy in flight). Process-wide; cycles <= 0 restores the default (about 0.2 s). A wait that runs out makes
 * the kernel return early with the status word set (moc_read_status / moc_publish_status report it); nothing traps
 * or spins forever. No counterpart in the reference. */
int moc_debug_set_wait_cycles(int64_t cycles);

/* Asynchronous form of the same check: enqueues a one-thread kernel on `stream` that copies the status word of
 * `workspace` to *host_word if it is non-zero. host_word must be pinned host memory that the device can address
 * (cudaHostAlloc / cudaMallocHost; with unified addressing its host pointer is valid on the device). The caller
 * polls *host_word from the host at its own pace; no synchronisation, no copy-engine transfer, capturable in a
 * CUDA graph. No counterpart in the reference (its kernels have no bounded waits). */
int moc_publish_status(const void* workspace, int* host_word, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOC_B200_H_ */
