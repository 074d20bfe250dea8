/*
 * nnue_b200.h -- C ABI of libnnue_b200.so, the sm_100a implementation of the
 * sparse feature-transformer hot path of nnue-pytorch.
 *
 * Conventions shared by every entry point
 *   - plain C: pointers, sizes and scalars only; no torch / C++ types.
 *   - every pointer is a DEVICE pointer owned by the caller unless the
 *     parameter name starts with `h_` (host).  Kernels that need scratch take
 *     a caller-provided workspace whose size the matching *_workspace_bytes()
 *     call returns.  What the library creates by itself, once per device, on
 *     the first call that needs it and kept until the process ends: a helper
 *     stream with two events (first backward call), 16 bytes of device memory
 *     plus 16 bytes of pinned host memory (first nnue_ft_fused_bwd call with
 *     mode = NNUE_BWD_AUTO), the timing events of nnue_b200_profile, and the
 *     fixed arrays of its device image (status words, norm partials, the
 *     scratch of nnue_ft_sparse_bwd_static).  Nothing else is allocated.
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default
 *     stream).  Work is only enqueued; nothing synchronises with the host.
 *   - the return value is a status: 0 (NNUE_OK) or a negative NNUE_ERR_*
 *     code.  nnue_b200_last_error() gives the message for the calling
 *     thread's most recent failure.  Nothing throws, traps or exits.
 *   - index lists follow the reference contract: int32, row-major [B, K],
 *     the first negative entry ends a row; duplicates are summed with
 *     multiplicity.  Entries >= N are skipped and recorded in the device
 *     status word (nnue_b200_device_status) instead of being dereferenced.
 *   - row widths: the vectorised kernels need W % 4 == 0 (and L1 % 8 == 0
 *     for the fused op) plus 16-byte aligned base pointers; other shapes run
 *     the scalar kernels of the same library.
 *
 * Citations name files of official-stockfish/nnue-pytorch by their path in
 * that project.
 */
#ifndef NNUE_B200_H
#define NNUE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NNUE_B200_ABI_VERSION 1

enum {
    NNUE_OK = 0,
    NNUE_ERR_ARG = -1,        /* null pointer, negative size, bad enum */
    NNUE_ERR_ALIGN = -2,      /* pointer not aligned as required */
    NNUE_ERR_WORKSPACE = -3,  /* workspace too small */
    NNUE_ERR_UNSUPPORTED = -4,/* shape outside what the kernels cover */
    NNUE_ERR_CUDA = -5,       /* a CUDA runtime call failed (message has it) */
    NNUE_ERR_INDEX = -6,      /* device status word reported bad indices */
    NNUE_ERR_TIMEOUT = -7     /* a bounded device-side wait ran out */
};

/* Scatter strategy of the backward kernels. */
enum {
    NNUE_BWD_AUTO = 0,     /* segment reduction, except that nnue_ft_fused_bwd switches to
                              atomics while the lists it saw on its previous auto call of the
                              same batch size held fewer than 6 active rows on average
                              (nearly empty boards; the count reaches the host without a
                              synchronisation, one call late) */
    NNUE_BWD_ATOMIC = 1,   /* vector red.global.add into a zeroed gradient */
    NNUE_BWD_SEGMENT = 2   /* CSR by row + gather-sum; every row written once */
};

int nnue_b200_abi_version(void);
const char* nnue_b200_last_error(void);

/* Number of kernels this process has launched through the library so far
 * (host-side tally, all devices). */
int64_t nnue_b200_launch_count(void);

/* Tuning knob for experiments ("fwd_u", "bwd_u", "stage_idx", ...).
 * Unknown keys return NNUE_ERR_ARG.  Process-wide, not thread-safe. */
int nnue_b200_tune(const char* key, int value);

/* Per-kernel device times of the calls made while profiling is on: the library
 * brackets its main kernels with CUDA events on the stream they run on.
 *   nnue_b200_profile(1)   clears the record and starts recording;
 *   nnue_b200_profile(0)   stops.
 *   nnue_b200_profile_read SYNCHRONISES the device, then returns entry i of
 *     the record grouped by kernel name (*h_name points at a string constant,
 *     *h_total_ms is the sum over its launches); NNUE_ERR_ARG past the end.
 * Process-wide, one host thread; events are created as needed and kept. */
int nnue_b200_profile(int32_t enable);
int nnue_b200_profile_read(int32_t i, const char** h_name, double* h_total_ms,
                           int64_t* h_launches);

/* L2 -> SM read probe: the access shape of the gather kernels without their
 * index lists and epilogue.  `buf` holds `rows` rows of 1024 bytes (16-byte
 * aligned; keep rows * 1 KiB well inside the L2 so that after one warm-up
 * launch every read is an L2 hit).  `warps` warps each sum `rows_per_warp`
 * rows (pattern 0: consecutive rows from a per-warp start; 1: pseudo-random
 * rows), every lane loading two 16-byte pieces per row with eight loads in
 * flight, and store one 16-byte result per lane to `sink`
 * (warps * 512 bytes).  Bytes read per launch: warps * rows_per_warp * 1024;
 * the caller times the launch with events on `stream`. */
int nnue_l2_read_probe(const void* buf, int64_t rows, int64_t warps,
                       int32_t rows_per_warp, int32_t pattern, void* sink,
                       void* stream);

/* Reads (and clears) the device status word.  SYNCHRONISES `stream`.
 * h_bad_index_count / h_timeout_count may be NULL.  Returns NNUE_OK,
 * NNUE_ERR_INDEX or NNUE_ERR_TIMEOUT. */
int nnue_b200_device_status(void* stream, int64_t* h_bad_index_count,
                            int64_t* h_timeout_count);

/* ---- A1: sparse linear forward ---------------------------------------
 * out[b, c] = bias[c] + sum_k weight[idx[b, k], c]   (bias first, k ascending)
 * Replaces the CuPy kernel `sparse_input_linear_forward`,
 * model/modules/feature_transformer/sparse_linear_kernel.py:114-157, launched
 * from model/modules/feature_transformer/sparse_linear_functions.py:78-101. */
int nnue_ft_sparse_fwd(const int32_t* idx, const float* weight,
                       const float* bias, float* out,
                       int64_t B, int32_t K, int64_t N, int32_t W,
                       void* stream);

/* ---- A2: sparse linear backward --------------------------------------
 * grad_weight[r, c] = sum over (b, k) with idx[b, k] == r of grad_out[b, c]
 * grad_bias[c]      = sum_b grad_out[b, c]
 * Both outputs are fully overwritten (no pre-zeroing by the caller).
 * Replaces `sparse_input_linear_backward`,
 * model/modules/feature_transformer/sparse_linear_kernel.py:237-288 and the
 * torch.zeros + launch in sparse_linear_functions.py:104-136. */
size_t nnue_ft_sparse_bwd_workspace_bytes(int64_t B, int32_t K, int64_t N,
                                          int32_t W, int32_t mode);
int nnue_ft_sparse_bwd(const int32_t* idx, const float* grad_out,
                       float* grad_weight, float* grad_bias,
                       int64_t B, int32_t K, int64_t N, int32_t W,
                       void* workspace, size_t workspace_bytes, int32_t mode,
                       void* stream);

/* ---- sparse linear backward without any allocation ---------------------
 * No counterpart in the reference project.
 * Same result as nnue_ft_sparse_bwd (segment route), for hosts that cannot
 * obtain a workspace because they must not allocate device memory when the
 * call is made: a process whose device memory is owned by its own pool, or a
 * service that forbids allocation after start-up.  The scratch is a fixed array of
 * NNUE_SPARSE_BWD_STATIC_SCRATCH_BYTES inside the library's device image
 * (every GPU that loads the library carries it until the process ends); the
 * call allocates nothing and frees nothing.
 *   - shapes whose scratch need (nnue_ft_sparse_bwd_workspace_bytes) exceeds
 *     the array are refused with NNUE_ERR_WORKSPACE and a message;
 *   - the first call on each device looks up the array's address
 *     (cudaGetSymbolAddress; with the CUDA runtime's lazy module loading this is
 *     also when the array's 32 MiB appear in device memory, the only time a
 *     call changes the amount of free memory); make that first call before any stream capture
 *     begins, and from one host thread (the per-device address cache is
 *     filled without a lock; concurrent first calls would only repeat the
 *     look-up);
 *   - all calls share the one array: two calls that can overlap on the GPU
 *     (different streams, no ordering between them) race on it.  Calls on one
 *     stream, or otherwise ordered, are safe; nothing has to be cleared by the
 *     caller between calls. */
#define NNUE_SPARSE_BWD_STATIC_SCRATCH_BYTES ((size_t)32 << 20)
int nnue_ft_sparse_bwd_static(const int32_t* idx, const float* grad_out,
                              float* grad_weight, float* grad_bias,
                              int64_t B, int32_t K, int64_t N, int32_t W,
                              void* stream);

/* ---- A6: fused double feature transformer, forward --------------------
 * Per position: w = bias[:L1] + sum weight[white_idx][:L1], b likewise;
 * x = us*[w, b] + them*[b, w] (2*L1 wide, four chunks of L1/2);
 * c = clamp(x, 0, max_act); l0 = [c0*c1, c2*c3];
 * wpsqt = bias[L1+p] + sum weight[white_idx][L1+p], bpsqt likewise,
 * p = psqt_idx[b].  `saved` [B, 4, L1/2] receives the PRE-clamp x, which is
 * what nnue_ft_fused_bwd consumes.  Optional epilogue, fused because it would
 * otherwise be several dense passes over l0: with act_quant_scale > 0,
 * l0 = floor(l0 * act_quant_scale + act_quant_eps) / act_quant_scale (the
 * reference's fake_quantize_ft_act, model/quantize.py:36-45, straight-through
 * in the backward), then l0 *= out_scale (its l0_correction_factor,
 * composed_feature_transformer.py:143-149).  Pass 0, 0, 1 for the bare op.
 * Replaces `fused_double_ft_forward`,
 * model/modules/feature_transformer/fused_ft_kernel.py:27-117, launched from
 * fused_ft_functions.py:47-75; numerics follow the torch composition in
 * double_ft_functions.py:62-80. */
int nnue_ft_fused_fwd(const float* us, const float* them,
                      const int32_t* white_idx, const int32_t* black_idx,
                      const int64_t* psqt_idx,
                      const float* weight, const float* bias, float max_act,
                      float act_quant_scale, float act_quant_eps, float out_scale,
                      float* l0, float* wpsqt, float* bpsqt, float* saved,
                      int64_t B, int32_t K, int64_t N, int32_t L1, int32_t P,
                      void* stream);

/* ---- A7: fused double feature transformer, backward -------------------
 * Gradient of the op above w.r.t. weight [N, L1+P] and bias [L1+P]; the
 * clamp passes gradient on the closed interval [0, max_act] like
 * torch.clamp.  Both outputs are fully overwritten.
 * Replaces `fused_double_ft_backward`,
 * model/modules/feature_transformer/fused_ft_kernel.py:147-272 and the
 * torch.zeros + launch in fused_ft_functions.py:81-122. */
size_t nnue_ft_fused_bwd_workspace_bytes(int64_t B, int32_t K, int64_t N,
                                         int32_t L1, int32_t P, int32_t mode);
int nnue_ft_fused_bwd(const float* us, const float* them,
                      const int32_t* white_idx, const int32_t* black_idx,
                      const int64_t* psqt_idx, float max_act, float out_scale,
                      const float* grad_l0, const float* grad_wpsqt,
                      const float* grad_bpsqt, const float* saved,
                      float* grad_weight, float* grad_bias,
                      int64_t B, int32_t K, int64_t N, int32_t L1, int32_t P,
                      void* workspace, size_t workspace_bytes, int32_t mode,
                      void* stream);

/* ---- A10/A11: table preparation --------------------------------------
 * out[r, c] = fq(weight[r, c] + virtual_weight[r % n_virtual, c]) in one pass,
 * fq(x) = round_half_even(x * s) / s with s = scale_main for c < L1 and
 * scale_psqt for the P PSQT columns; virtual_weight may be NULL (no folding),
 * scale_main <= 0 switches the quantization off.  Replaces the dense passes of
 * model/modules/features/halfka_v2_hm.py:68-69 (weight + virtual.repeat) and
 * model/modules/feature_transformer/composed_feature_transformer.py:61-76
 * (two fake-quantizations and a concat).  The gradient of `out` is the
 * gradient of `weight` unchanged (straight-through); the factor rows receive
 * nnue_ft_virtual_grad: out[v, c] = sum_b grad[b * n_virtual + v, c]. */
int nnue_ft_prepare_table(const float* weight, const float* virtual_weight,
                          float* out, int64_t N, int64_t n_virtual,
                          int32_t L1, int32_t P, float scale_main,
                          float scale_psqt, void* stream);
int nnue_ft_virtual_grad(const float* grad, float* out, int64_t N,
                         int64_t n_virtual, int32_t W, void* stream);

/* ---- N1, integer form: the forward on an int16 table --------------------------
 * With weight fake quantization on, every L1 entry of the table the operator
 * reads is k / scale_main with integer k (scale_main = 256 in the reference,
 * model/quantize.py:58-73).  nnue_ft_quantize_table writes that table as
 *   q16  int16 [N, L1]   k = round_half_even((weight + virtual_weight[r % n_virtual]) * scale_main), columns
 *                        (c, c + 1), c even, stored together as the int32 number k[c + 1] * 65536 + k[c];
 *                        rows q16_pitch elements apart (a multiple of 8, >= L1).  The forward wants ONE MORE
 *                        row behind the table, row N, all zeros (the caller clears it): padding and
 *                        out-of-range list entries read it, which keeps the gather loop free of branches
 *   psqt float [N, P]    the PSQT columns, fake-quantized at scale_psqt as nnue_ft_prepare_table does
 * and updates d_stats (two device int32 the caller zeroes before the first block of a table):
 * d_stats[0] += entries with |k| > 32767 (stored saturated), d_stats[1] = max(d_stats[1], max |k|).
 * nnue_ft_fused_fwd_q16 is nnue_ft_fused_fwd on that table: integer sums of the k (column pairs summed
 * as one 32-bit number and split every 32767 / d_stats[1] rows), one multiplication by 1 / scale_main,
 * then the same epilogue (a table with d_stats[1] > 4095, weights above 16.0, also takes the fp32 route).  The results are bit for bit those of nnue_ft_fused_fwd on the table
 * nnue_ft_prepare_table makes from the same parameters: with |k| <= 32767 and K <= 511 no partial sum of the
 * fp32 form is ever rounded.  `bias_fq` is the bias as that forward takes it (fp32 [L1 + P], its L1 part
 * fake-quantized at scale_main; quantize it into the same d_stats as a one-row table so that its range
 * counts).  While d_stats[0] != 0 the kernel ignores q16 and gathers
 * round((weight + virtual) * scale_main) / scale_main from the parameter blocks themselves (h_blocks: the
 * table's row ranges in order, their `rows` adding up to N), so the results never depend on the range; the
 * host does not have to read the words.  d_stats may hold n_stat_parts such pairs (parts of the table quantized
 * by different kernels or ranks): any overflow counts, the largest max |k| rules.  A block whose `weight` is NULL
 * has no fp32 parameters to fall back to (a data-parallel rank that only receives integer rows): the route is
 * then refused and tallied in the device status word.  Needs L1 % 16 == 0, P % 4 == 0, K <= 511, a power-of-two
 * scale_main.
 * Replaces the same reference code as nnue_ft_prepare_table + nnue_ft_fused_fwd. */
typedef struct nnue_ft_block {
    const float* weight;          /* [rows, L1 + P] */
    const float* virtual_weight;  /* [n_virtual, L1 + P] or NULL */
    int64_t rows;
    int64_t n_virtual;
} nnue_ft_block;

int nnue_ft_quantize_table(const float* weight, const float* virtual_weight,
                           int16_t* q16, int64_t q16_pitch, float* psqt, int64_t N, int64_t n_virtual,
                           int32_t L1, int32_t P, float scale_main, float scale_psqt,
                           int32_t* d_stats, void* stream);

/* The bias of nnue_ft_fused_fwd_q16 in one small launch: bias_fq[0, L1) = round(bias * scale_main) / scale_main (the
 * bits nnue_ft_prepare_table gives), bias_fq[L1, L1 + P) = 0, and the range statistics of the L1 part (entries beyond
 * int16, max |k|) added to d_stats[0..1] or, with overwrite_stats != 0, written over them. */
int nnue_ft_prepare_bias_q16(const float* bias, float* bias_fq, int32_t L1, int32_t P, float scale_main,
                             int32_t* d_stats, int32_t overwrite_stats, void* stream);
int nnue_ft_fused_fwd_q16(const float* us, const float* them,
                          const int32_t* white_idx, const int32_t* black_idx,
                          const int64_t* psqt_idx, const int16_t* q16, int64_t q16_pitch, const float* psqt,
                          const float* bias_fq, float scale_main, const int32_t* d_stats, int32_t n_stat_parts,
                          const nnue_ft_block* h_blocks, int32_t n_blocks,
                          float max_act, float act_quant_scale, float act_quant_eps, float out_scale,
                          float* l0, float* wpsqt, float* bpsqt, float* saved,
                          int64_t B, int32_t K, int64_t N, int32_t L1, int32_t P, void* stream);

/* The same backward with the gradient delivered in row slices, for a consumer
 * on another stream (the data-parallel reduce) that starts on the first rows
 * while the later ones are still computed.  h_slices->row_bounds holds
 * n_slices + 1 non-decreasing rows, the first 0 and the last N; rows
 * [bounds[i], bounds[i+1]) are final when events[i] (a cudaEvent_t or NULL) is
 * recorded on the call's stream.  The values written are those of the unsliced
 * call, bit for bit.  The setting belongs to this one call: nothing is kept
 * between calls.  Every successful return has recorded every event exactly
 * once, also on the routes that finish the whole gradient at once (B == 0,
 * mode = NNUE_BWD_ATOMIC; NNUE_BWD_AUTO with slices is the segment route).
 * h_slices == NULL or n_slices == 0 is nnue_ft_fused_bwd.
 *
 * by_columns != 0 slices the gradient by COLUMNS instead: row_bounds then holds
 * column bounds in floats, the first 0 and the last L1 + P, every inner bound a
 * multiple of nnue_ft_fused_bwd_column_tile(L1, P); columns [bounds[i], bounds[i+1])
 * of ALL rows are final when events[i] is recorded.  The gather-sum walks the
 * table's columns tile by tile anyway, so column slices cost it nothing (row
 * slices make it read its scratch once per slice). */
#define NNUE_BWD_MAX_SLICES 16
typedef struct nnue_bwd_slices {
    int32_t n_slices;
    int64_t row_bounds[NNUE_BWD_MAX_SLICES + 1];
    void* events[NNUE_BWD_MAX_SLICES];
    int32_t by_columns;
} nnue_bwd_slices;

/* Width in floats of the column tiles of the segment route at this shape under the current tuning (0 when the
 * shape takes the scalar route, which cannot be sliced). */
int32_t nnue_ft_fused_bwd_column_tile(int32_t L1, int32_t P);

int nnue_ft_fused_bwd_sliced(const float* us, const float* them,
                             const int32_t* white_idx, const int32_t* black_idx,
                             const int64_t* psqt_idx, float max_act, float out_scale,
                             const float* grad_l0, const float* grad_wpsqt,
                             const float* grad_bpsqt, const float* saved,
                             float* grad_weight, float* grad_bias,
                             int64_t B, int32_t K, int64_t N, int32_t L1, int32_t P,
                             void* workspace, size_t workspace_bytes, int32_t mode,
                             const nnue_bwd_slices* h_slices, void* stream);

/* ---- A12: RangerLite (Adam + positive-negative momentum + lookahead) ---
 * One fused pass over a parameter tensor viewed as [rows, width]:
 *   g  = grad * (*d_grad_scale if given) ;
 *   vm = beta2*vm + (1-beta2)*g*g ; denom = sqrt(vm)/sqrt(bc2) + eps ;
 *   pnm:  pos = (step odd ? grad_ma : neg_grad_ma) ;
 *         pos = beta1^2*pos + (1-beta1^2)*g ;
 *         upd = ((1+f)*pos - f*neg) * (1/noise_norm) ;
 *   adam: grad_ma = beta1*grad_ma + (1-beta1)*g ; upd = grad_ma ;
 *   p = p*wd_keep - step_size*upd/denom ;
 *   if merge: p = alpha*p + (1-alpha)*slow ; slow = p.
 * `row_active` (optional, uint8 [rows]) implements the touched-rows-only
 * update: a row whose flag is 0 and whose gradient row is entirely zero is
 * skipped (bit-identical, because all of its moments are still zero); a row
 * with any non-zero gradient gets its flag set for good.
 * Replaces the five CuPy kernels of model/optimizers/ranger_lite.py:46-201,
 * the per-tensor launches at :325-477 and the lookahead pass at :746-768;
 * the arithmetic follows the Python path at :592-742. */
typedef struct nnue_ranger_hparams {
    /* every constant is derived on the host in double precision, as the
     * reference's Python code does, and rounded to float once */
    float beta2;
    float one_minus_beta2;
    float mom;             /* beta1^2 with PNM, beta1 without */
    float one_minus_mom;
    float one_plus_f;      /* 1 + pnm_momentum */
    float f;               /* pnm_momentum */
    float noise_norm_inv;  /* 1/sqrt((1+f)^2 + f^2) */
    float step_size;       /* lr / bias_correction1 */
    float bc2_sqrt;        /* sqrt(1 - beta2^step) */
    float eps;
    float wd_keep;         /* 1 - decay*lr/variance_norm; 1 = no decay */
    float alpha;           /* lookahead blending */
    float one_minus_alpha;
    int32_t use_pnm;       /* 1 = PNM, 0 = plain Adam */
    int32_t step_is_odd;   /* PNM buffer selection */
    int32_t do_merge;      /* 1 = lookahead merge in the same pass */
    int32_t phase;         /* 0 = full update, 1 = second moment only,
                              2 = update reading the stored second moment */
} nnue_ranger_hparams;

int nnue_rangerlite_update(float* p, const float* grad, float* grad_ma,
                           float* neg_grad_ma, float* variance_ma, float* slow,
                           uint8_t* row_active, const float* d_grad_scale,
                           int64_t rows, int64_t width,
                           const nnue_ranger_hparams* h_hp, void* stream);

/* The same update that also leaves the new parameter values as the integer table of
 * nnue_ft_quantize_table (q16 with `rows` rows + the caller's zero row, psqt, d_stats: zeroed by this call,
 * then the overflow count and max |k| of ALL rows, updated or not), for a [rows, L1 + P] table without
 * factor rows.  The next forward then needs no pass of its own over the table. */
typedef struct nnue_table_emit {
    int16_t* q16;
    int64_t q16_pitch;
    float* psqt;
    int32_t* d_stats;
    int32_t L1, P;
    float scale_main, scale_psqt;
} nnue_table_emit;

int nnue_rangerlite_update_emit(float* p, const float* grad, float* grad_ma,
                                float* neg_grad_ma, float* variance_ma, float* slow,
                                uint8_t* row_active, const float* d_grad_scale,
                                int64_t rows, int64_t width,
                                const nnue_ranger_hparams* h_hp, const nnue_table_emit* h_emit,
                                void* stream);

/* Standalone lookahead merge, model/optimizers/ranger_lite.py:746-768. */
int nnue_lookahead_merge(float* p, float* slow, int64_t n, float alpha,
                         void* stream);

/* Sum of squares of a gradient tensor into *d_out (accumulating, so several
 * tensors can share one scalar), and the clip coefficient
 * prescale * min(1, max_norm / (prescale * sqrt(*d_sumsq) + 1e-6)) that
 * torch.nn.utils.clip_grad_norm_ applies at trainer/engine.py:308-311.
 * `prescale` is 1, or 1/world when the gradients are rank SUMS that still
 * have to become means (the division rides in the coefficient). */
int nnue_grad_sumsq(const float* grad, int64_t n, float* d_out_sumsq,
                    void* stream);
/* Both norm entry points (and the norm inside nnue_ddp_reduce_shard) add their
 * per-CTA partial sums in a fixed order, so the result is reproducible run to
 * run; the partials live in a file-scope device array of the library, which
 * calls overlapping on the GPU (different streams) must not share. */
int nnue_clip_coef(const float* d_sumsq, float max_norm, float prescale,
                   float* d_coef, void* stream);

/* Several tensors per launch (at most NNUE_MULTI_MAX per launch; longer lists
 * are split).  Same arithmetic as nnue_grad_sumsq / nnue_rangerlite_update
 * (no row flags); each tensor carries its own constants, as each of the
 * trainer's ten parameter groups (model/nnue.py:117-182) may differ.  The
 * arrays are HOST arrays; their contents are copied into the launch. */
#define NNUE_MULTI_MAX 16
typedef struct nnue_ranger_tensor {
    float* p;
    const float* grad;
    float* grad_ma;
    float* neg_grad_ma;   /* NULL unless hp.use_pnm */
    float* variance_ma;
    float* slow;          /* NULL unless hp.do_merge */
    int64_t n;
    nnue_ranger_hparams hp;
} nnue_ranger_tensor;

int nnue_grad_sumsq_multi(const float* const* h_grads, const int64_t* h_n,
                          int32_t count, float* d_out_sumsq, void* stream);
int nnue_rangerlite_update_multi(const nnue_ranger_tensor* h_tensors,
                                 int32_t count, const float* d_grad_scale,
                                 void* stream);

/* ---- A14: data-parallel exchange fused with the optimizer ----------------
 * Replaces, for the feature-transformer table, the DistributedDataParallel
 * all-reduce of trainer/engine.py:149-162 followed by a full optimizer step on
 * every rank.  h_*_ptrs are HOST arrays of `world` DEVICE pointers: the same
 * [N*W] float buffer on every rank, mapped into this process (symmetric memory
 * or CUDA IPC).  [elem_begin, elem_end) is this rank's shard in elements
 * (multiples of 4).  Plain peer loads/stores only.
 *   nnue_ddp_reduce_shard: own_grad[i] = sum_r grad_r[i] (rank order) for the
 *     shard, and *d_sumsq += sum of squares of those sums.
 *   nnue_ddp_update_shard: RangerLite (nnue_rangerlite_update arithmetic,
 *     phase 0) on the shard, reading `grad` (this rank's buffer, full size)
 *     and shard-sized moment tensors, and storing the new values into every
 *     rank's table.
 * The caller orders the ranks: every rank's backward before any reduce, every
 * reduce before the next backward, every update before the next forward (a
 * small NCCL collective on the same stream between the phases does it). */
int nnue_ddp_reduce_shard(float* const* h_grad_ptrs, int32_t world, int32_t rank,
                          int64_t elem_begin, int64_t elem_end, float* d_sumsq,
                          void* stream);
int nnue_ddp_update_shard(float* const* h_table_ptrs, int32_t world, int32_t rank,
                          int64_t elem_begin, int64_t elem_end, const float* grad,
                          float* grad_ma, float* neg_grad_ma, float* variance_ma,
                          float* slow, const float* d_grad_scale,
                          const nnue_ranger_hparams* h_hp, void* stream);

/* nnue_ddp_reduce_shard over a 2-D block of the gradient viewed as [rows, width]: rows [row_begin, row_end), columns
 * [col_begin, col_end) (floats, multiples of 4).  With the backward delivering column slices
 * (nnue_bwd_slices.by_columns), a rank reduces that slice of its own rows while later columns are computed. */
int nnue_ddp_reduce_block(float* const* h_grad_ptrs, int32_t world, int32_t rank, int64_t row_begin,
                          int64_t row_end, int64_t col_begin, int64_t col_end, int64_t width,
                          float* d_sumsq, void* stream);

/* nnue_ddp_update_shard that also (or instead) sends the other ranks what their next forward gathers: the
 * rows of the integer table (nnue_ft_quantize_table's format) written into EVERY rank's int16 and PSQT
 * tables with plain peer stores.  With fp32_to_peers = 0 the fp32 rows stay with their owner: half the bytes
 * cross NVLink, and the other ranks' fp32 tables go stale outside their own share until the caller gathers them
 * (checkpoints, evaluation through the fp32 table).  d_stats_local (device int32[2], zeroed by the caller before the
 * first call of a step) collects the overflow count and max |k| of this rank's share; nnue_ddp_publish_stats then
 * stores the pair into slot `rank` of every rank's statistics array (int32 [2 * world]), which the forward reads
 * as `n_stat_parts = world` parts. */
typedef struct nnue_ddp_emit {
    int16_t* const* h_q16_ptrs;    /* host array of `world` device pointers */
    float* const* h_psqt_ptrs;
    int32_t* const* h_stats_ptrs;
    int32_t* d_stats_local;
    int64_t q16_pitch;
    int32_t L1, P;
    float scale_main, scale_psqt;
    int32_t fp32_to_peers;
} nnue_ddp_emit;

int nnue_ddp_update_shard_emit(float* const* h_table_ptrs, int32_t world, int32_t rank,
                               int64_t elem_begin, int64_t elem_end, const float* grad,
                               float* grad_ma, float* neg_grad_ma, float* variance_ma,
                               float* slow, const float* d_grad_scale,
                               const nnue_ranger_hparams* h_hp, const nnue_ddp_emit* h_emit,
                               void* stream);
int nnue_ddp_publish_stats(const nnue_ddp_emit* h_emit, int32_t world, int32_t rank, void* stream);

/* ---- layer stack behind the feature transformer --------------------------
 * Bucket-aware replacement of the three wide F.linear calls + row selection of
 * model/modules/stacked_linear.py:38-66 and of the activation / skip / output
 * quantization code of model/modules/layer_stacks.py:33-84: only the weight
 * block of a position's own bucket is multiplied.  L2 = L3 = 32, L1 % 32 == 0,
 * at most 16 buckets.  Weight layouts are the reference's (after factor merge
 * and fake quantization, which stay with the caller): W1 [C*32, L1], b1 [C*32],
 * W2 [C*32, 64], b2 [C*32], W3 [C, 128], b3 [C].
 *   nnue_ls_plan      groups the batch by bucket into tiles (stable); `plan`
 *                     is caller memory of nnue_ls_plan_bytes(B, C) bytes and is
 *                     shared by the forward and backward calls of one batch.
 *   nnue_ls_l1_fwd    o1 [B, 32] = W1[bucket] x + b1[bucket]
 *   nnue_ls_l1_bwd    dx [B, L1] (skipped when NULL), dW1, db1 (overwritten)
 *   nnue_ls_tail_fwd  y [B] and the saved pre-activations o2 [B, 32]
 *   nnue_ls_tail_bwd  d_o1 [B, 32], dW2, db2, dW3, db3 (overwritten) */
typedef struct nnue_ls_params {
    float act_scale;      /* hidden_quantized_one (128); 0 = no activation fake quantization */
    float act_eps;        /* 1e-5 */
    float sqr_corr;       /* sqr_crelu_correction_factor */
    float max_hidden;     /* hidden_quantized_max / hidden_quantized_one */
    float out_den;        /* 2 * hidden_one * weight_scale_l_out (32768) */
    float out_mul;        /* nnue2score * weight_scale_out (9600) */
    int32_t quantize_out; /* 1 = output fake quantization (truncating division) */
} nnue_ls_params;

size_t nnue_ls_plan_bytes(int64_t B, int32_t C);
int nnue_ls_plan(const int64_t* bucket, int64_t B, int32_t C, void* plan,
                 size_t plan_bytes, void* stream);
int nnue_ls_l1_fwd(const float* x, const float* W1, const float* b1,
                   const void* plan, float* o1, int64_t B, int32_t L1, int32_t C,
                   void* stream);
/* nnue_ls_l1_fwd on the tensor cores (tcgen05.mma kind::tf32, accumulator in tensor memory), for inputs TF32
 * holds exactly: x on the activation grid (q / 128, q <= 127) and W1 fake-quantized (k / 128, |k| < 2048), which
 * is what the quantized model feeds this layer.  Products and partial sums are then exact and the result has the
 * bits of nnue_ls_l1_fwd; other inputs are truncated to TF32 on the way in.  Same arguments. */
int nnue_ls_l1_fwd_tc(const float* x, const float* W1, const float* b1,
                      const void* plan, float* o1, int64_t B, int32_t L1, int32_t C,
                      void* stream);
int nnue_ls_l1_bwd(const float* x, const float* W1, const float* d_o1,
                   const void* plan, float* dx, float* dW1, float* db1,
                   int64_t B, int32_t L1, int32_t C, void* stream);
/* nnue_ls_l1_bwd with the INPUT gradient on the tensor cores, for W1 that TF32 holds exactly (the quantized model):
 * d_o1 is split into three TF32-exact parts (hi + mid + lo = d_o1, every subtraction exact), so every product the
 * tensor core forms is exact and only the fp32 accumulation of its 96 terms rounds (not the bits of the FMA kernel:
 * another summation order; 1e-6 of the tensor's max-norm).  The weight and bias gradients come from the FMA kernel
 * (their sums run over the whole batch).  Needs L1 %% 128 == 0 and nnue_ls_l1_bwd_tc_workspace_bytes(L1, C) bytes of
 * scratch (the transposed weights); dx == NULL is nnue_ls_l1_bwd. */
size_t nnue_ls_l1_bwd_tc_workspace_bytes(int32_t L1, int32_t C);
int nnue_ls_l1_bwd_tc(const float* x, const float* W1, const float* d_o1,
                      const void* plan, float* dx, float* dW1, float* db1,
                      int64_t B, int32_t L1, int32_t C, void* workspace,
                      size_t workspace_bytes, void* stream);
int nnue_ls_tail_fwd(const float* o1, const void* plan, const float* W2,
                     const float* b2, const float* W3, const float* b3,
                     const nnue_ls_params* h_params, float* o2, float* y,
                     int64_t B, int32_t C, void* stream);
size_t nnue_ls_tail_bwd_workspace_bytes(int64_t B, int32_t C);
int nnue_ls_tail_bwd(const float* o1, const float* o2, const void* plan,
                     const float* W2, const float* W3, const float* grad_y,
                     const nnue_ls_params* h_params, float* d_o1, float* dW2,
                     float* db2, float* dW3, float* db3, void* workspace,
                     size_t workspace_bytes, int64_t B, int32_t C, void* stream);

/* Effective layer-stack weights of one step, all six tensors in one launch:
 * w1 = fq(l1_w + repeat(l1f_w, C)), b1 likewise (model/modules/stacked_linear.py:96-127),
 * w2, b2, w3, b3 = fq of their parameters, fq(v) = round_half_even(v * scale) / scale
 * when scales.quantize (model/quantize.py:49-50), else v.  l1f_w / l1f_b may both be NULL.
 * Shapes: l1_w [C*32, L1], l1_b [C*32], l1f_w [32, L1], l1f_b [32], l2_w [C*32, 64],
 * l2_b [C*32], out_w [C, 128], out_b [C]; outputs alike.
 * The straight-through backward is the identity on every tensor plus
 * nnue_ls_fold_grads: d_l1f_w = sum over buckets of dW1 (bucket order), d_l1f_b likewise. */
typedef struct nnue_ls_weight_scales {
    float w1, b1, w2, b2, w3, b3;
    int32_t quantize;
} nnue_ls_weight_scales;

int nnue_ls_effective_weights(const float* l1_w, const float* l1_b,
                              const float* l1f_w, const float* l1f_b,
                              const float* l2_w, const float* l2_b,
                              const float* out_w, const float* out_b,
                              const nnue_ls_weight_scales* h_scales,
                              float* w1, float* b1, float* w2, float* b2,
                              float* w3, float* b3, int32_t L1, int32_t C,
                              void* stream);
int nnue_ls_fold_grads(const float* dW1, const float* db1, float* d_l1f_w,
                       float* d_l1f_b, int32_t L1, int32_t C, void* stream);

/* ---- Q: integer quantized evaluation ----------------------------------
 * Integer restatement of the fake-quantized forward defined by
 * model/quantize.py:36-56,133-147, model/modules/layer_stacks.py:33-84 and
 * model/model.py:107-133.  The reference holds no integer evaluator; this is
 * the arithmetic an engine performs on the exported net.
 * Weights: ft_w int16 [N, L1], ft_psqt int32 [N, P], ft_b int32 [L1] (bias at
 * the ft scale), l1_w int8 [buckets, L2, L1] + l1_b int32 [buckets, L2],
 * l2_w int8 [buckets, L3, 2*L2] + l2_b, out_w int8 [buckets, 2*L2+2*L3] +
 * out_b int32 [buckets].  `out` int32 [B] is the evaluation in units of
 * 1/(2*nnue2score*weight_scale_out) of the float model output. */
typedef struct nnue_quant_params {
    int32_t ft_max;        /* 255 */
    int32_t ft_shift;      /* 9: (c0*c1) >> 9 */
    int32_t hidden_max;    /* 127 */
    int32_t sqr_shift_l1;  /* 21 */
    int32_t sqr_eps_l1;    /* 20 */
    int32_t lin_shift_l1;  /* 7 */
    int32_t sqr_shift_l2;  /* 19 */
    int32_t sqr_eps_l2;    /* 5 */
    int32_t lin_shift_l2;  /* 6 */
    int32_t skip_mul;      /* (hidden_one*ws_l_out)/(hidden_one*ws_l1) = 1 */
    int32_t out_mul;       /* 9600 = nnue2score*weight_scale_out */
    int32_t out_div;       /* 32768 = 2*hidden_one*weight_scale_l_out */
} nnue_quant_params;

int nnue_quant_eval(const int32_t* white_idx, const int32_t* black_idx,
                    const uint8_t* stm_white, const int32_t* bucket,
                    const int16_t* ft_w, const int32_t* ft_psqt,
                    const int32_t* ft_b,
                    const int8_t* l1_w, const int32_t* l1_b,
                    const int8_t* l2_w, const int32_t* l2_b,
                    const int8_t* out_w, const int32_t* out_b,
                    int32_t* out,
                    int64_t B, int32_t K, int64_t N, int32_t L1, int32_t L2,
                    int32_t L3, int32_t P, int32_t buckets,
                    const nnue_quant_params* h_qp, void* stream);

/* The same evaluation in two kernels: the feature-transformer part as a gather
 * whose table slice stays in the L2 (column tiles are the slow grid dimension,
 * as in nnue_ft_fused_fwd), then the layers.  Results are bit-identical to
 * nnue_quant_eval; it needs nnue_quant_eval_workspace_bytes(B, L1) bytes of
 * scratch (less is accepted: the batch is then processed in more passes) and
 * ft_b 16-byte aligned. */
size_t nnue_quant_eval_workspace_bytes(int64_t B, int32_t L1);
int nnue_quant_eval_tiled(const int32_t* white_idx, const int32_t* black_idx,
                          const uint8_t* stm_white, const int32_t* bucket,
                          const int16_t* ft_w, const int32_t* ft_psqt,
                          const int32_t* ft_b,
                          const int8_t* l1_w, const int32_t* l1_b,
                          const int8_t* l2_w, const int32_t* l2_b,
                          const int8_t* out_w, const int32_t* out_b,
                          int32_t* out,
                          int64_t B, int32_t K, int64_t N, int32_t L1, int32_t L2,
                          int32_t L3, int32_t P, int32_t buckets,
                          const nnue_quant_params* h_qp, void* workspace,
                          size_t workspace_bytes, void* stream);

/* The tiled evaluation on a PACKED copy of the feature-transformer table, for nets whose |ft_w| <= 4095 (trained
 * nets are far below): nnue_quant_pack_table writes int16 [N + 1, L1] in which every pair of neighbouring columns is
 * the int32 number ft_w[c + 1] * 65536 + ft_w[c] (a negative low value borrows from the high half) and the last row
 * is zero, and leaves max |ft_w| in *d_max_abs (device int32; the caller reads it once and passes it on).  The gather
 * then adds two columns per 32-bit add with a branch-free row loop (padding reads the zero row), a warp per
 * (position, perspective).  Bit-identical to nnue_quant_eval_tiled; refused when max_abs > 4095 or K > 511. */
int nnue_quant_pack_table(const int16_t* ft_w, int16_t* packed, int32_t* d_max_abs, int64_t N, int32_t L1,
                          void* stream);
int nnue_quant_eval_packed(const int32_t* white_idx, const int32_t* black_idx,
                           const uint8_t* stm_white, const int32_t* bucket,
                           const int16_t* ft_w_packed, int32_t max_abs,
                           const int32_t* ft_psqt, const int32_t* ft_b,
                           const int8_t* l1_w, const int32_t* l1_b,
                           const int8_t* l2_w, const int32_t* l2_b,
                           const int8_t* out_w, const int32_t* out_b,
                           int32_t* out,
                           int64_t B, int32_t K, int64_t N, int32_t L1, int32_t L2,
                           int32_t L3, int32_t P, int32_t buckets,
                           const nnue_quant_params* h_qp, void* workspace,
                           size_t workspace_bytes, void* stream);

/* ---- L: training loss and its gradient, one launch ------------------------
 * `calculate_sf_loss` with `remap_tablebase_score` (model/nnue.py:18-69), fused
 * with the PSQT term of the model output (model/model.py:107-133) and the
 * scaling to centipawns:
 *   net_i = y_i + (wpsqt_i - bpsqt_i) * (us_i - 0.5)      (PSQT inputs may be NULL)
 *   loss  = sum_i w_i |pt_i - qf(net_i * net_scale)|^pow_exp / sum_i w_i
 * `loss` is a device scalar.  d_y (and d_wpsqt, d_bpsqt), when not NULL,
 * receive d loss / d y (d wpsqt, d bpsqt), float [B].  `workspace` holds
 * nnue_sf_loss_workspace_bytes() bytes, 8-byte aligned, zeroed once by the
 * caller before the first call and left zeroed by every call; two calls that
 * share a workspace must not overlap on the GPU.  All sums run in a fixed order. */
typedef struct nnue_loss_params {
    float in_offset, out_offset;      /* 270, 270 */
    float in_scaling, out_scaling;    /* 340, 380 */
    float pow_exp;                    /* 2.5 */
    float qp_asymmetry;               /* 0 */
    float w1, w2;                     /* 0, 0.5 */
    float tb_remap_base, tb_remap_scale, tb_remap_decay; /* 4000, 4000, 0.85 */
    float lambda;                     /* weight of the search score against the game outcome */
    float net_scale;                  /* nnue2score = 600 */
} nnue_loss_params;

size_t nnue_sf_loss_workspace_bytes(void);
int nnue_sf_loss(const float* y, const float* wpsqt, const float* bpsqt,
                 const float* us, const float* score, const float* outcome,
                 const nnue_loss_params* h_params, float* loss, float* d_y,
                 float* d_wpsqt, float* d_bpsqt, void* workspace, int64_t B,
                 void* stream);

/* ---- N3: device-side batch construction ----------------------------------
 * Replaces the CPU fill of `SparseBatch` (data_loader/cpp/training_data_loader.cpp:29-73)
 * and the shipping of expanded index lists (data_loader/_native.py:48-96): the
 * host ships one 72-byte record per position, the GPU writes the tensors that
 * `get_tensors` returns.  Index formula: model/modules/features/halfka_v2_hm.py:8-36.
 *
 * piece[s]: bits 0-5 square (0 = a1, 63 = h8), bits 6-8 piece type 1..6
 * (P N B R Q K), bit 9 = white piece.  Slots >= count are ignored.  Lists are
 * written in slot order and padded with -1.
 * NNUE_LAYOUT_NATIVE: 12 piece planes, rows [0, 24576), K >= 32.
 * NNUE_LAYOUT_FLAT:   11 planes (kings share plane 10): the `count` real rows
 * [0, 22528), then the `count` matching factor rows [22528, 23232), K >= 64.
 * us/them/outcome/score are float [B]; piece_count and bucket_idx
 * ((count-1)/4, the PSQT / layer-stack bucket) are int64 [B] and may be NULL.
 * A record with a count outside 2..32, a piece type outside 1..6, an outcome
 * above 2, or not exactly one king per side is tallied in the device status
 * word and yields two empty lists. */
typedef struct nnue_packed_position {
    uint16_t piece[32];
    int16_t score;      /* centipawns */
    uint8_t outcome2;   /* game result x 2: 0, 1, 2 */
    uint8_t stm_white;  /* 1 = white to move */
    uint8_t count;      /* pieces on the board, 2..32 */
    uint8_t pad[3];
} nnue_packed_position;

enum { NNUE_LAYOUT_NATIVE = 0, NNUE_LAYOUT_FLAT = 1 };

int nnue_batch_build_halfka(const nnue_packed_position* positions, int64_t B,
                            int32_t layout, int32_t K, int32_t* white_idx,
                            int32_t* black_idx, float* us, float* them,
                            float* outcome, float* score, int64_t* piece_count,
                            int64_t* bucket_idx, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NNUE_B200_H */
