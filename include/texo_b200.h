/*
 * C ABI of the B200 quantized-matmul library.
 *
 * Two packagings of the same operators are built:
 *
 *   libmm_int8.so, libmm_int4.so, libdequantization.so, librms_norm_w_residual.so
 *       each exports the single symbol `solve` with exactly the prototype the reference
 *       declares for that operator, so tests/mm_int8.cpp, tests/mm_int4.cpp and
 *       tests/dequantization.cpp of frezcirno/Texo link against them unchanged
 *       (libmm_int4a8.so follows the same convention for an operator the reference lacks).
 *
 *   libtexo_b200.so
 *       all of them in one library; the sources are compiled with -Dsolve=<name>, the
 *       reference's own convention for co-linking operators (its Makefile:129-148), giving
 *       the texo_*_solve names below, plus the entry points without a reference counterpart.
 *
 * Common contract (reference docs/operators.md:9-12, src/mm_int8.cu:530-592): every pointer
 * is a DEVICE pointer owned by the caller, row-major and contiguous; inputs are never
 * written; the output is fully overwritten and nothing outside it is touched; work is
 * issued asynchronously on the legacy default stream of the current device and the
 * functions return void - poll cudaGetLastError() and synchronise before reading results.
 * Scratch memory is owned by the library (per device, grow-only, never freed).  Calls are
 * not thread-safe.
 */
#ifndef TEXO_B200_H
#define TEXO_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- combined library: libtexo_b200.so ---------------------------------------------- */

/* INT8 zero-point/scale matmul.  Replaces `solve` of the reference's src/mm_int8.cu:530-535
 * (declared by its harness at tests/mm_int8.cpp:5-6).  A [M,K], B [K,N], C [M,N] int8.
 *   C = clamp(rint(float(sum_k (A-zA)(B-zB)) * scale_A * scale_B / scale_C) + zC, -128, 127)
 * with the FP32 operation order of src/mm_int8.cu:12-25.  M, N > 0; K >= 0; with K == 0,
 * A and B may be null and C is filled with clamp(zero_point_C).  Any byte alignment. */
void texo_mm_int8_solve(const int8_t* A, const int8_t* B, int8_t* C, int M, int N, int K,
                        float scale_A, float scale_B, float scale_C, int zero_point_A,
                        int zero_point_B, int zero_point_C);

/* W4A16 weight-only matmul.  Replaces `solve` of the reference's src/mm_int4.cu:386-390
 * (tests/mm_int4.cpp:7-8).  x [M,K] fp16, w_q [N,K/2] uint8 (high nibble = even k, value =
 * nibble - 8), scales [N,K/group_size] fp16, y [M,N] fp16; fp16 passed as 16-bit words.
 * M <= 0 or N <= 0 is a no-op (src/mm_int4.cu:391-392). */
void texo_mm_int4_solve(const void* x, const uint8_t* w_q, const void* scales, void* y, int M,
                        int N, int K, int group_size);

/* Allocation-free form of texo_mm_int8_solve.  It has no counterpart in the reference (whose
 * solve always goes through a cudaMalloc'd scratch, src/mm_int8.cu:500-509).  For callers
 * that may not allocate device memory while running - HBM fully handed to their own pools,
 * or a loop that cannot take the device-wide stall of cudaMalloc/cudaFree.  The scratch is
 * a fixed 256 KiB array inside the library image on every GPU that loads it; limits
 * M <= 32768 and N <= 32768.  Returns 0, or -1 bad arguments, -2 size beyond the limits,
 * -3 device set-up failed.  Same results as texo_mm_int8_solve.  First call per device does
 * a one-time set-up (make it outside stream capture); calls share the scratch, so calls
 * that would overlap on the GPU race. */
int texo_mm_int8_solve_noalloc(const int8_t* A, const int8_t* B, int8_t* C, int M, int N, int K,
                               float scale_A, float scale_B, float scale_C, int zero_point_A,
                               int zero_point_B, int zero_point_C);
/* Error state of texo_mm_int8_solve_noalloc on the current device, read without allocating
 * (no counterpart in the reference; texo_mm_int8_status is not for these callers, its status
 * block is cudaMalloc'd).  0 = all such calls since the last query completed; 1-5 = a bounded
 * device-side wait gave up in one of them and its C is incomplete; -3 = device set-up failed.
 * Blocking 4-byte copy out of the fixed scratch array; clears the word when it was set. */
int texo_mm_int8_noalloc_status(void);

/* Host-buffer form of texo_mm_int8_solve: A, B, C are HOST pointers (pinned for full speed).
 * Does what the reference harness does around `solve` (upload, run, download:
 * tests/mm_int8.cpp:56-79) as a pipeline of row chunks on internal streams, so uploads,
 * compute and downloads overlap.  Asynchronous; C_host is valid after
 * cudaDeviceSynchronize().  Returns 0, -1 bad arguments, -3 CUDA failure. */
int texo_mm_int8_solve_host(const int8_t* A_host, const int8_t* B_host, int8_t* C_host, int M, int N,
                            int K, float scale_A, float scale_B, float scale_C, int zero_point_A,
                            int zero_point_B, int zero_point_C);

/* Prepared weights for mm_int8 (no counterpart in the reference, which recomputes colsum(B)
 * and a transposed copy of B on every call, src/mm_int8.cu:559-561).  prepare() computes
 * colsum(B) once for a device-resident B [K,N] (asynchronously, default stream) and returns
 * a handle; solve_prepared() is texo_mm_int8_solve with B, K, N taken from the handle and
 * only the row sums of the new activations left to compute; results are bit-identical.  B
 * must stay alive and unchanged until release().  prepare() returns NULL on bad arguments. */
typedef struct texo_int8_weights texo_int8_weights;
texo_int8_weights* texo_mm_int8_prepare_weights(const int8_t* B, int K, int N);
void texo_mm_int8_release_weights(texo_int8_weights* weights);
void texo_mm_int8_solve_prepared(const int8_t* A, const texo_int8_weights* weights, int8_t* C, int M,
                                 float scale_A, float scale_B, float scale_C, int zero_point_A,
                                 int zero_point_B, int zero_point_C);
/* texo_mm_int8_solve_prepared with rowsum(A) supplied as well: row_sum_A [M] int32 (device),
 * row m = sum_k A[m,k], e.g. as written by texo_rms_norm_quant_solve.  With the column sums
 * in the handle and the row sums from the producer, a call launches the tensor kernel alone.
 * row_sum_A null = texo_mm_int8_solve_prepared. */
void texo_mm_int8_solve_presummed(const int8_t* A, const int* row_sum_A, const texo_int8_weights* w,
                                  int8_t* C, int M, float scale_A, float scale_B, float scale_C,
                                  int zero_point_A, int zero_point_B, int zero_point_C);

/* Tile-scale dequantization.  Replaces `solve` of the reference's
 * src/dequantization.cu:40-43 (tests/dequantization.cpp:4).  X, Y [M,N] fp32,
 * S [ceil(M/T), ceil(N/T)] fp32; Y = X * S[m/T][n/T]. */
void texo_dequantization_solve(const float* X, const float* S, float* Y, int M, int N, int T);

/* ---- diagnostics (no counterpart in the reference, whose operators return void and keep no
 * error state; see reference tests/test_utils.h:11-17 for its only error handling) ------- */

/* mm_int8 with per-output-channel weight quantisation (no counterpart in the reference, which
 * is per-tensor only, src/mm_int8.cu:533-535): scale_B [N] FP32 and zero_point_B [N] int32 are
 * DEVICE arrays, zero_point_B may be null (all zero).  Column n:
 *   C[m,n] = clamp(rint(float(sum_k (A-zA)(B-zB[n])) * scale_A * scale_B[n] / scale_C) + zC)
 * in the FP32 operation order of texo_mm_int8_solve.  Arrays 16-byte aligned for the
 * tensor-core paths (otherwise the generic kernel runs). */
void texo_mm_int8_solve_per_channel(const int8_t* A, const int8_t* B, int8_t* C, int M, int N, int K,
                                    float scale_A, const float* scale_B, float scale_C,
                                    int zero_point_A, const int* zero_point_B, int zero_point_C);

/* mm_int8 with per-group weight scales (no counterpart in the reference: its INT8 operator is
 * per-tensor, src/mm_int8.cu:533-535; its per-group scheme is the FP16 one of
 * src/mm_int4.cu:309-317): scale_B [K / group_size, N] FP32 on the device, one scale per scale
 * group of group_size consecutive k and output column; group_size divides K.  With dot_g the
 * exact integer dot of group g:
 *   acc = 0; for g ascending: acc = fma(RN(float(dot_g) * scale_A), scale_B[g, n], acc)  (FP32)
 *   C[m, n] = clamp(rint(acc / scale_C) + zero_point_C, -128, 127)
 * (one group = the per-channel form).  Runs a SIMT kernel on every shape. */
void texo_mm_int8_solve_per_group(const int8_t* A, const int8_t* B, int8_t* C, int M, int N, int K,
                                  int group_size, float scale_A, const float* scale_B, float scale_C,
                                  int zero_point_A, int zero_point_B, int zero_point_C);
/* The same for packed-INT4 weights: scale_B [N, K / group_size] FP32 on the device (the layout of
 * the reference's W4A16 scales, src/mm_int4.cu:5-6, in FP32). */
void texo_mm_int4a8_solve_per_group(const int8_t* A, const uint8_t* w_q, int8_t* C, int M, int N, int K,
                                    int group_size, float scale_A, const float* scale_B, float scale_C,
                                    int zero_point_A, int zero_point_B, int zero_point_C);

/* Gate/up projection with the SwiGLU consumer fused into the epilogue (no counterpart in the
 * reference as one operator; it fuses its INT8 matmul, src/mm_int8.cu, with the formula of its
 * src/swiglu.cu:15-18).  B_gu [K, 2F] int8 holds gate and up weight columns interleaved
 * (column 2j = gate j, 2j+1 = up j); H [M, F] int8:
 *   gate = float(dot_gate) * scale_A * scale_gate,  up = float(dot_up) * scale_A * scale_up,
 *   H = clamp(rint(up * gate / (1 + exp(-gate)) / scale_H) + zero_point_H, -128, 127)
 * with the dots as in texo_mm_int8_solve (zero points zero_point_gate / zero_point_up for the
 * two kinds of column).  exp is the GPU's approximate __expf, as in the reference operator. */
void texo_mm_int8_swiglu_solve(const int8_t* A, const int8_t* B_gu, int8_t* H, int M, int F, int K,
                               float scale_A, float scale_gate, float scale_up, float scale_H,
                               int zero_point_A, int zero_point_gate, int zero_point_up,
                               int zero_point_H);

/* INT8 matmul with a dequantising drain (the reference reaches the same values with mm_int8
 * into an int8 C followed by a separate dequantisation pass; fused here, no counterpart as
 * one operator): Y [M,N] FP16 (16-bit words) = half(float(dot) * scale_A * scale_B) with
 * dot = sum_k (A-zA)(B-zB) exact, the two FP32 multiplies in this order, one round-to-nearest
 * conversion to FP16. */
void texo_mm_int8_dequant_solve(const int8_t* A, const int8_t* B, void* Y, int M, int N, int K,
                                float scale_A, float scale_B, int zero_point_A, int zero_point_B);

/* mm_int8 on one GPU's column slab of the weights with the all-gather of C fused into the
 * epilogue (the reference has no multi-GPU code).  C_all is a HOST array of n_gpus (<= 8)
 * DEVICE pointers: entry r is GPU r's copy of the full output [M, ld_c], this process's own
 * copy and peer mappings of the others (torch symmetric memory, CUDA IPC, cuMem).  The call
 * computes C[:, col_offset : col_offset + N_slab] from A [M,K] and B_slab [K,N_slab] exactly
 * as texo_mm_int8_solve and stores every finished piece into all n_gpus copies (plain stores
 * over NVLink, no multicast, no waiting on other GPUs).  After all GPUs' calls have completed
 * and the caller has synchronised them, every copy holds the whole C.  Returns 0, or -1 for
 * invalid arguments. */
int texo_mm_int8_solve_allgather(const int8_t* A, const int8_t* B_slab, int8_t* const* C_all,
                                 int n_gpus, int M, int N_slab, int K, int ld_c, int col_offset,
                                 float scale_A, float scale_B, float scale_C, int zero_point_A,
                                 int zero_point_B, int zero_point_C);
/* The same with the NVLink multicast (NVLS) mapping of that allocation as well (no reference
 * counterpart): C_multicast is the multicast address of the [M, ld_c] matrix (torch symmetric
 * memory handle.multicast_ptr + the tensor's offset, or a cuMem multicast mapping), 16-byte
 * aligned, or null.  With it each whole 128-byte row segment leaves this GPU once
 * (multimem.st, replicated by NVSwitch into every copy) instead of once per peer. */
int texo_mm_int8_solve_allgather_multicast(const int8_t* A, const int8_t* B_slab, int8_t* const* C_all,
                                           int8_t* C_multicast, int n_gpus, int M, int N_slab, int K,
                                           int ld_c, int col_offset, float scale_A, float scale_B,
                                           float scale_C, int zero_point_A, int zero_point_B,
                                           int zero_point_C);

/* W4A8: packed-INT4 weights against INT8 activations, INT8 output.  No counterpart in the
 * reference (its mm_int4 takes FP16 activations, src/mm_int4.cu:386-390); it combines the
 * reference's weight format - w_q [N,K/2] uint8, high nibble = even k, value = nibble - 8
 * (src/mm_int4.cu:5-6,25-26) - with the arithmetic and argument meaning of its INT8 operator
 * (src/mm_int8.cu:12-25,530-535):
 *   C[m,n] = clamp(rint(float(sum_k (A[m,k]-zA)(q[n,k]-zB)) * sA * sB / sC) + zC, -128, 127)
 * A [M,K] int8, C [M,N] int8, device pointers, legacy default stream, asynchronous.  K even,
 * K >= 0 (K == 0: A and w_q may be null); any byte alignment (the tensor-core path needs
 * 16-byte aligned A / w_q and K % 32 == 0, other calls take a SIMT kernel). */
void texo_mm_int4a8_solve(const int8_t* A, const uint8_t* w_q, int8_t* C, int M, int N, int K,
                          float scale_A, float scale_B, float scale_C, int zero_point_A,
                          int zero_point_B, int zero_point_C);
/* W4A8 with per-output-channel weight quantisation (no counterpart in the reference): scale_B
 * [N] FP32 and zero_point_B [N] int32 (each within [-128, 127]) are DEVICE arrays, one entry
 * per row of w_q; zero_point_B may be null (all zero).  Column n:
 *   C[m,n] = clamp(rint(float(sum_k (A-zA)(q[n,k]-zB[n])) * scale_A * scale_B[n] / scale_C) + zC)
 * in the FP32 operation order of texo_mm_int4a8_solve.  Arrays 16-byte aligned and N % 4 == 0
 * for the tensor-core paths (otherwise the generic kernel runs). */
void texo_mm_int4a8_solve_per_channel(const int8_t* A, const uint8_t* w_q, int8_t* C, int M, int N,
                                      int K, float scale_A, const float* scale_B, float scale_C,
                                      int zero_point_A, const int* zero_point_B, int zero_point_C);
/* mm_int4a8 diagnostics: path 1 = generic SIMT kernel, 2 = tcgen05 kind::i8 CTA-pair kernel,
 * 3 = TMA + tcgen05 streaming kernel (M <= 32), 4 = register-streaming decode kernel (M <= 16,
 * K % 128 == 0, aligned A / w_q): packed weights read once from HBM straight into registers,
 * mma.sync s8 x u8. */
int texo_mm_int4a8_last_path(void);
void texo_mm_int4a8_force_path(int path);
int texo_mm_int4a8_status(void);

/* RMSNorm with residual add, FP32.  Replaces `solve` of the reference's
 * src/rms_norm_w_residual.cu:66-75: x, residual, out [N,C], weight [C], device pointers,
 *   out = (x + residual) * rsqrt(mean_j((x + residual)^2) + eps) * weight.
 * The sum of squares is reduced in FP32 in this library's own (fixed) order, as the
 * reference reduces it in its own: results agree to FP32 reduction error. */
void texo_rms_norm_w_residual_solve(const float* x, const float* residual, const float* weight,
                                    float* out, int N, int C, float eps);
/* The same, fused with INT8 activation quantisation - the producer of mm_int8's A.  No
 * counterpart in the reference.  q [N,C] int8 = clamp(rint(out / scale) + zero_point, -128,
 * 127) with `out` as above (never written to memory); z_out [N,C] FP32, if not null, receives
 * x + residual (the updated residual stream); q_row_sum [N] int32, if not null, receives
 * sum_j q[n,j] for texo_mm_int8_solve_presummed.  scale finite and non-zero. */
void texo_rms_norm_quant_solve(const float* x, const float* residual, const float* weight,
                               int8_t* q, float* z_out, int* q_row_sum, int N, int C, float eps,
                               float scale, int zero_point);
/* 1 = two-pass kernel (any C, any alignment), 2 = row-in-registers kernel (C % 4 == 0,
 * C <= 16384, 16-byte aligned pointers). */
int texo_rms_norm_last_path(void);

/* Which device path the last mm_int8 call took (also the SwiGLU and FP16 forms): 1 generic,
 * 2 one-CTA tensor kernel (tcgen05), 3 skinny (streaming, M <= 128), 4 CTA-pair tensor kernel. */
int texo_mm_int8_last_path(void);
/* Force a path for the following calls (0 = automatic).  A forced path is still skipped
 * when its preconditions do not hold.  Also settable with TEXO_MM_INT8_PATH. */
void texo_mm_int8_force_path(int path);
/* Reads and clears the error state of the current device: 0 = none, 1-5 = a bounded
 * device-side wait gave up (kernel returned early, results invalid), 16 = bad argument,
 * 17 = tensor-map creation failed (call fell back to the generic path), 18 = a kernel launch
 * was refused (call fell back to the generic path).  Synchronises.  After a non-zero device
 * code (1-5) the split-K workspace of the decode path is re-zeroed here, so poll this after
 * any suspected failure before trusting later decode-shaped results. */
int texo_mm_int8_status(void);

/* mm_int4: 1 = generic FP32 kernel, 2 = tcgen05 kind::f16 CTA-pair kernel with a TMEM drain
 * per scale group (needs 16-byte aligned x / w_q, K % 64 == 0, group_size 16, 32, 64 or 128),
 * 4 = the same pipeline with the scale folded exactly into the weight operand (FP16 hi + lo,
 * two MMAs per k step, one drain per tile; the default for group_size <= 64),
 * 3 = streaming (decode) kernel
 * (M <= 16, group_size 128, K % 128 == 0, aligned x / w_q): packed weights read once from HBM
 * straight into registers, mma.sync on 16-row activation tiles. */
int texo_mm_int4_last_path(void);
void texo_mm_int4_force_path(int path);
int texo_mm_int4_status(void);

/* Failure-path self-test: makes one device-side bounded wait run out of its budget (about a
 * second) on a barrier nothing completes, and returns the status code the kernel recorded
 * (5), or a negative value if the kernel did not return normally.  Nothing faults or hangs. */
int texo_selftest_wait_timeout(void);

/* Hits / misses of the library's cache of encoded TMA descriptors (a call with a pointer and
 * shape seen before skips the driver's descriptor encoding); either pointer may be null. */
void texo_tensor_map_cache_stats(long long* hits, long long* misses);

/* Sets the per-device epoch counter with which the CTA-pair kernels (mm_int8, mm_int4a8) mark
 * finished row / column sums (diagnostic, no reference counterpart): lets a test drive the
 * counter across its 32-bit wrap, where the library clears the flags. */
void texo_set_sums_epoch(unsigned value);

/* Number of kernels the library has launched so far in this process. */
long long texo_kernel_launches(void);
/* CUDA-event bracket around the dominant kernel of each following call (for roofline
 * reporting).  enable(1) resets the record; read() synchronises and returns the summed
 * kernel time and the number of bracketed launches (0 on success). */
void texo_profile_enable(int on);
int texo_profile_read(float* total_ms, int* launches);

/* Tensor-pipe ceiling probe (no counterpart in the reference): issues kind::i8 MMAs back to
 * back on shared-memory-resident operands, `batches` x 64 instructions per SM (pairs = 0) or
 * per SM pair (pairs = 1), and returns the achieved tera-ops per second, negative on error.
 * Used by the benchmark as the box-measured INT8 denominator.  Synchronises. */
double texo_int8_issue_ceiling_tops(int pairs, int batches);
/* Same with `per_commit` MMAs between tcgen05.commit signals instead of 64. */
double texo_int8_issue_rate_tops(int pairs, int batches, int per_commit);
/* The same probe with kind::f16 MMAs; tera-flops per second. */
double texo_f16_issue_rate_tflops(int pairs, int batches, int per_commit);
/* Operand-feed probe: streams the TMA boxes of an INT8 GEMM over A [M,K], B [K,N] (device
 * pointers, 16-byte aligned rows) through a ring of `stages` (1..7) shared-memory stages
 * without computing; returns TB/s of operand bytes delivered to the SMs.  mode bit 0 = A
 * boxes, bit 1 = B boxes.  Synchronises. */
double texo_int8_feed_rate_tbs(const void* A, const void* B, int M, int N, int K, int stages,
                               int mode);

#ifdef __cplusplus
}
#endif
#endif /* TEXO_B200_H */
