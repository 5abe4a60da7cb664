/*
 * sparseforge_b200 — C ABI of the B200 (sm_100a) SparseLinear hot path.
 *
 * Every entry point takes raw device pointers, explicit sizes, dtype enums, scalar
 * hyper-parameters and a CUDA stream (passed as void*, 0 = legacy default stream).
 * No torch type crosses this boundary. The caller allocates and owns every buffer,
 * outputs and scratch included; the library keeps no pointer after a call returns.
 * All work is enqueued on the given stream; no entry point synchronises the device.
 *
 * Return value: 0 on success, a negative sf_status on failure (nothing is launched
 * after a failed argument check). sf_last_error_string() returns the message of the
 * last failure on the calling thread.
 *
 * Each declaration cites the interface of the SparseForge reference
 * (liuhanzuo/SparseForge, paths relative to that project) that it stands in for.
 */
#ifndef SPARSEFORGE_B200_H
#define SPARSEFORGE_B200_H

#include <stdint.h>

#if defined(__GNUC__)
#define SF_API __attribute__((visibility("default")))
#else
#define SF_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    SF_OK = 0,
    SF_ERR_BAD_ARG = -1,      /* null pointer, negative size, unknown enum */
    SF_ERR_UNSUPPORTED = -2,  /* valid but not implemented (dtype / shape combination) */
    SF_ERR_ALIGNMENT = -3,    /* pointer or leading dimension not aligned as required */
    SF_ERR_CUDA = -4,         /* a CUDA runtime / driver call failed */
    SF_ERR_DEVICE_WAIT = -5   /* a bounded device-side wait ran out (see sf_gemm_status) */
} sf_status;

typedef enum { SF_F32 = 0, SF_BF16 = 1, SF_I8 = 2 } sf_dtype;

/* Importance metrics of compute_gate_target, legacy/sparse_modeling.py:1041-1079. */
typedef enum {
    SF_METRIC_HESSIAN_OBD = 0,   /* (H + 1e-8) * W^2 */
    SF_METRIC_HESSIAN_RATIO = 1, /* |W| / sqrt(H + 1e-8) */
    SF_METRIC_MAGNITUDE = 2,     /* |W| */
    SF_METRIC_HESSIAN = 3,       /* H */
    SF_METRIC_MOVEMENT = 4       /* |W * grad_ema| / temperature (aux = grad_ema) */
} sf_metric;

/* Penalty pull inside update_mask, legacy/sparse_modeling.py:1295-1573. */
typedef enum {
    SF_PENALTY_NONE = 0,
    SF_PENALTY_TOPN = 1, /* 'nm_2_4' (:1350-1393) and 'structured_topn' (:1532-1566) */
    SF_PENALTY_MID = 2   /* 'mid' (:1567-1570) */
} sf_penalty_mode;

/* Hard view of a soft mask in the general N:M entry points. */
typedef enum {
    SF_HARD_TOPN = 0,     /* top N of every group of M ('structured', legacy/sparse_modeling.py:720-735) */
    SF_HARD_THRESHOLD = 1 /* mask > 0.5 ('unstructured', :526-527); N:M then only shapes beta mixing and the top-N pull */
} sf_hard_view;

SF_API int sf_version(void);
SF_API const char* sf_last_error_string(void);

/* Number of doubles of scratch sf_hutch_score needs for `n` weight elements. */
SF_API int64_t sf_hutch_score_scratch_doubles(int64_t n);

/*
 * Hutchinson Hessian-diagonal accumulation fused with the importance score and the
 * layer-wide score statistics.
 *   replaces: update_hessian_hutchinson elementwise tail, legacy/utils.py:804-868
 *             score formulas, legacy/sparse_modeling.py:1041-1079
 *             mean / population std of the score, legacy/sparse_modeling.py:1084-1088
 *   if hvp != NULL:  H <- beta*H + (1-beta)*max(hvp*v, 0)      (H fp32, in place)
 *   score <- metric(W, H)                                      (fp32, raw)
 *   norm[0] <- mean(score), norm[1] <- std_pop(score) + 1e-6   (fp32, on device)
 * hvp and W have dtype w_dtype; v has dtype v_dtype (SF_I8 holding +1 / -1 only, or w_dtype).
 * aux is grad_ema for SF_METRIC_MOVEMENT (w_dtype), else ignored; aux_scalar is the
 * movement temperature. scratch: sf_hutch_score_scratch_doubles(n) doubles.
 * n = rows*cols, must be a multiple of 8; buffers 16-byte aligned.
 * On return scratch[0] and scratch[1] hold sum(score) and sum(score^2) of this call, for
 * callers that hold one shard of a layer and combine the sums across shards.
 */
SF_API int sf_hutch_score(const void* hvp, const void* v, int v_dtype, float* H, const void* W,
                   int w_dtype, const void* aux, double aux_scalar, float* score,
                   float* norm, double* scratch, int64_t n, double beta, int metric,
                   void* stream);

/*
 * norm <- (mean, std_pop + 1e-6) from sums[0] = sum(score), sums[1] = sum(score^2) over n
 * elements (device pointers). Used after the sums of the row shards of one layer have been
 * added up across ranks; the same arithmetic as the tail of sf_hutch_score
 * (legacy/sparse_modeling.py:1085-1087 over the whole layer).
 */
SF_API int sf_score_norm_from_sums(const double* sums, double n, float* norm, void* stream);

/*
 * Gradient EMA and g^2 Hessian proxy of SparseLinear.update_grad_hessian_ema
 * (legacy/sparse_modeling.py:901-922) in one pass over the gradient:
 *   grad_ema <- b * grad_ema + (1 - b) * g                      (g, grad_ema in `dtype`)
 *   H        <- b * H + (1 - b) * round_dtype(g * g)            (H fp32; skipped when H is NULL)
 * with ATen's rounding points (mul_ rounds to the tensor dtype, add_ with alpha is one fused step).
 * n is a multiple of 8, every buffer 16-byte aligned. The early return of the reference for
 * layers without a grad_ema tensor (every metric but `movement`) is the caller's.
 */
SF_API int sf_grad_hessian_ema(const void* g, void* grad_ema, int dtype, float* H, int64_t n, double beta,
                               void* stream);

/*
 * sf_hutch_score without a scratch argument: the partial sums go to an array that is part
 * of the library image. This entry point has no counterpart in the reference. It is for
 * callers that are not allowed to allocate device memory at the point where they need the
 * score, for example a hook that runs in the middle of a training step while a caching
 * allocator owns all free memory and a cudaMalloc would stall or fail, code that must not
 * cause the implicit device synchronisation of cudaMalloc / cudaFree, or a process that runs
 * under a fixed device-memory budget. The call allocates nothing, on the device or through
 * any library. Inputs and outputs are still the caller's buffers, as in sf_hutch_score.
 *
 * Limits and rules:
 *  - The array is 4096 doubles (32 KiB), resident on every GPU that loads the library until
 *    the process ends: two partial sums for each of at most 2048 thread blocks. The grid is
 *    capped at 2048 blocks that stride over the input, so the array is large enough for any
 *    n; the limit SF_HUTCH_SCORE_STATIC_MAX_N (67,108,864 elements; the largest LLaMA-2-7B
 *    matrix has 45,088,768) is a fixed bound of this entry point, chosen so that what it
 *    accepts is stated and tested, not a capacity of the array. A larger n returns
 *    SF_ERR_UNSUPPORTED and launches nothing; use sf_hutch_score with your own scratch then.
 *  - The first call on each device looks up the array's device address (once per device,
 *    with that device current). Make that first call outside any CUDA stream capture.
 *  - All calls on one device share the array. It still holds the previous call's partial
 *    sums when the next call starts; that is harmless because each call overwrites every
 *    slot it later reads, and nothing needs to start at zero. Two calls that run on the GPU
 *    at the same time (different streams) would overwrite each other's sums: serialise them.
 */
#define SF_HUTCH_SCORE_STATIC_MAX_N ((int64_t)67108864)
SF_API int64_t sf_hutch_score_static_max_n(void);
SF_API int sf_hutch_score_static(const void* hvp, const void* v, int v_dtype, float* H, const void* W,
                                 int w_dtype, const void* aux, double aux_scalar, float* score,
                                 float* norm, int64_t n, double beta, int metric, void* stream);

/* Stats written by sf_mask_update_nm24 (8 doubles). */
enum {
    SF_MSTAT_FLIPS = 0,       /* sum xor(hard(prev mask), hard(new mask)), :1659-1661 */
    SF_MSTAT_SUM_M = 1,       /* sum m */
    SF_MSTAT_SUM_M1M = 2,     /* sum m(1-m)  (mid_penalty numerator, legacy/utils.py:913) */
    SF_MSTAT_SUM_TOP2 = 3,    /* sum of the two largest m per group (nm_2_4_tile_stats) */
    SF_MSTAT_SUM_BOT2 = 4,    /* sum of the two smallest m per group */
    SF_MSTAT_COUNT_LT_HALF = 5, /* count m < 0.5 (sparsity_penalty threshold path) */
    SF_MSTAT_COUNT = 8
};

/*
 * One structured (N:M = 2:4) soft-mask update with everything that depends on the new
 * mask, in one pass over the layer.
 *   replaces: SparseLinear.update_mask, legacy/sparse_modeling.py:1242-1666, with
 *             compute_gate_target structured branch :1084-1088, :1164-1185,
 *             beta mixing :1199-1225, penalty :1350-1393 / :1532-1570, binarize push
 *             :1575-1590, EMA :1593, flip count :1659-1661;
 *             effective mask of SparseLinear.forward :759-771 and the weight*mask of
 *             FusedMaskedLinearSTE.forward :74-81; _hard_mask_from_soft :720-735.
 *   s  = (score - norm[0]) / norm[1]   (rounded to bf16 first when score_bf16 != 0)
 *   G  = sigmoid((s - tau_g)/(T + 1e-8)), tau_g = 2nd largest s of the group of 4
 *        (or the exact 0/1 top-2 indicator when structured_exact != 0);
 *        with tau != NULL (device scalar, normalised-score units) the gate is the unstructured
 *        one of :1099-1162, G = sigmoid((s - *tau)/(T + 1e-8)), tau being the sampled quantile
 *        of _tau_unstructured :987-1015; everything after the gate is unchanged
 *   G  = (1-beta_s) G + beta_s top2(s)                      if beta_s > 0
 *   G  = clamp(G - pen*(mask - top2(G)), 0, 1)              SF_PENALTY_TOPN, pen != 0
 *   G  = clamp(G - pen*(1 - 2 mask), 0, 1)                  SF_PENALTY_MID,  pen != 0
 *   G  = G*(1-d) if G<0.5, G*(1+d) if G>0.5                 if d != 0
 *   mask <- clamp(mask*(1-a) + a*G, 0, 1)                   (fp32, in place)
 *   hard = top2(mask); M_eff = hx*mask + (1-hx)*hard (hx >= 1: mask itself)
 *   wm   <- W * cast(M_eff)   (w_dtype, optional)           meta <- 2:4 metadata of hard
 * Ties inside a group go to the lower column index everywhere.
 * meta: one byte per two groups, row-major [rows, cols/8]: low nibble = group 2j, high
 * nibble = group 2j+1; nibble = i0 | (i1 << 2) with i0 < i1 the kept column offsets.
 * stats: SF_MSTAT_COUNT doubles, overwritten. cols % 8 == 0.
 */
SF_API int sf_mask_update_nm24(const float* score, const float* norm, const float* tau, float* mask,
                        const void* W, int w_dtype, void* wm, uint8_t* meta, double* stats, int64_t rows,
                        int64_t cols, double temperature, double mask_lr, double pen,
                        int penalty_mode, double beta_s, double binarize_decay, double hx,
                        int structured_exact, int score_bf16, void* stream);

/*
 * sf_mask_update_nm24 without a score tensor: the score is formed again inside the pass from the
 * weight and the Hessian diagonal (metric SF_METRIC_HESSIAN_OBD, _HESSIAN_RATIO, _MAGNITUDE or
 * _HESSIAN; the same arithmetic as sf_hutch_score / sf_adamw_masked_score, so the result equals
 * the update from their score tensor bit for bit). The pass reads W anyway to write the masked
 * weight, so the optimizer pass before it need not write the score (score = NULL there) and this
 * pass reads H instead: 4 bytes per element less traffic per step. norm comes from
 * sf_adamw_masked_score / sf_hutch_score; wm and meta are required. No bf16 score rounding
 * (the metrics with a fp32 Hessian never need it).
 */
SF_API int sf_mask_update_nm24_from_weight(const void* W, int w_dtype, const float* H, int metric,
                                    const float* norm, const float* tau, float* mask, void* wm,
                                    uint8_t* meta, double* stats, int64_t rows, int64_t cols,
                                    double temperature, double mask_lr, double pen, int penalty_mode,
                                    double beta_s, double binarize_decay, double hx, int structured_exact,
                                    void* stream);

/*
 * sf_mask_update_nm24 with freeze bands (freeze_low > 0 or freeze_high < 1 in the layer config).
 *   replaces: the frozen-entry rule of compute_gate_target, legacy/sparse_modeling.py:1227-1229
 *             (a frozen entry's gate is its own value), and the snap at the end of update_mask,
 *             :1621-1642: after the update, entries <= freeze_low become 0 and, when apply_high
 *             (the reference applies it from step 2000 on), entries >= freeze_high become 1; the
 *             snapped entries are flagged. Projection, masked weight, metadata, flip count and
 *             sums see the snapped mask, as the reference's do.
 * frozen_flags: [rows, cols] fp32, 0 or 1, read and updated in place (flags only ever rise).
 */
SF_API int sf_mask_update_nm24_frozen(const float* score, const float* norm, const float* tau,
                               float* frozen_flags, double freeze_low, double freeze_high, int apply_high,
                               float* mask, const void* W, int w_dtype, void* wm, uint8_t* meta,
                               double* stats, int64_t rows, int64_t cols, double temperature,
                               double mask_lr, double pen, int penalty_mode, double beta_s,
                               double binarize_decay, double hx, int structured_exact, int score_bf16,
                               void* stream);

/*
 * WANDA importance metric: per-input-channel activation energy and the score built from it.
 *   replaces: SparseLinear.add_batch, legacy/sparse_modeling.py:884-898 (called from the calibration
 *             hooks of legacy/utils.py:2045-2047), and the 'wanda' branch of compute_gate_target,
 *             legacy/sparse_modeling.py:1071-1077, with the score statistics of :1084-1088.
 * sf_wanda_add_batch: scaler_row[c] <- scaler_row[c] * keep, then + ||x[:, c]||_2^2 / denom, both
 *   rounded to s_dtype as the two in-place tensor operations are. x: [rows, cols] of x_dtype (the
 *   batch flattened to tokens), cols % 8 == 0. The caller keeps nsamples on the host and passes
 *   keep = nsamples / (nsamples + batch + 1e-8) and denom = max(nsamples + batch, 1).
 *   scratch: sf_wanda_scratch_floats(cols) floats; the column sums are formed in a fixed order.
 * sf_wanda_score: score[r, c] <- |W[r, c]| * sqrt(scaler_row[c] + eps) (fp32 output; arithmetic
 *   rounded to bf16 after every operation where both operands are bf16), norm <- (mean, population
 *   std + 1e-6); scratch as for sf_hutch_score (scratch[0], scratch[1] = the two sums).
 */
SF_API int64_t sf_wanda_scratch_floats(int64_t cols);
SF_API int sf_wanda_add_batch(const void* x, int x_dtype, int64_t rows, int64_t cols, void* scaler_row,
                       int s_dtype, double keep, double denom, float* scratch, void* stream);
SF_API int sf_wanda_score(const void* W, int w_dtype, const void* scaler_row, int s_dtype, int64_t rows,
                   int64_t cols, double eps, float* score, float* norm, double* scratch, void* stream);

/*
 * Joint mask update of a GLU gate / up pair: both layers are updated from ONE score, the sum of
 * their importance scores, so that the same positions are pruned in both.
 *   replaces: _update_glu_joint_mask legacy/utils.py:363-479 with _compute_joint_gate_target
 *             :536-613 and _apply_mid_penalty_to_gate :616-643.
 * sf_score_sum: out <- a + b (fp32 scores of the two layers, e.g. written by sf_hutch_score) with
 *   norm <- (mean, population std + 1e-6) of out; scratch as for sf_hutch_score.
 * sf_mask_update_nm24_joint: sf_mask_update_nm24 with the penalty pull taken from `pen_mask`
 *   instead of the mask being updated (the reference forms the penalised gate once, from the
 *   gate layer's mask, and applies it to both layers); pen_mask = NULL is sf_mask_update_nm24.
 *   Call it once per layer with the joint score.
 */
SF_API int sf_score_sum(const float* a, const float* b, float* out, float* norm, double* scratch, int64_t n,
                 void* stream);
SF_API int sf_mask_update_nm24_joint(const float* score, const float* norm, const float* tau,
                              const float* pen_mask, float* mask, const void* W, int w_dtype, void* wm,
                              uint8_t* meta, double* stats, int64_t rows, int64_t cols, double temperature,
                              double mask_lr, double pen, int penalty_mode, double beta_s,
                              double binarize_decay, double hx, int structured_exact, int score_bf16,
                              void* stream);

/*
 * Hard top-2-of-4 projection along the input dimension.
 *   replaces: SparseLinear._hard_mask_from_soft 'nm_2_4' :578-603 and 'structured'
 *             :720-735, legacy/sparse_modeling.py; the inline copy at
 *             legacy/main_llama.py:2610-2661.
 * soft: [rows, cols] of dtype in_dtype with row stride ld_soft (elements). hard (optional)
 * gets 0/1 in out_dtype with row stride ld_hard; columns beyond (cols/4)*4 are 1.
 * meta (optional) as in sf_mask_update_nm24 with row stride ceil(cols/8) bytes.
 */
SF_API int sf_project_nm24(const void* soft, int in_dtype, int64_t ld_soft, void* hard, int out_dtype,
                    int64_t ld_hard, uint8_t* meta, int64_t rows, int64_t cols, void* stream);

/*
 * Effective masked weight without a mask update.
 *   replaces: SparseLinear.forward :759-771 + FusedMaskedLinearSTE.forward :74-81,
 *             legacy/sparse_modeling.py (there recomputed on every forward call).
 *   wm <- W * cast(hx*mask + (1-hx)*top2(mask));  finalized != 0 or hx >= 1: W * cast(mask).
 *   scale != 1 multiplies wm afterwards (weight_scaling, :777-784).
 */
SF_API int sf_effective_weight(const void* W, int w_dtype, const float* mask, void* wm, uint8_t* meta,
                        int64_t rows, int64_t cols, double hx, int finalized, double scale,
                        void* stream);

/*
 * Mask-aware AdamW step for one parameter tensor.
 *   replaces: AdamW.step, legacy/adamw.py:65-176 (order of operations as there):
 *   p *= 1 - lr*wd;  g += decay * p * (1 - mask)  (mask != NULL);
 *   m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2;  denom = sqrt(v)/sqrt(bc2) + eps;
 *   p -= (lr/bc1) m/denom;  p -= lr*l1*sign(p)/denom  (l1 > 0, mask != NULL).
 * bc1 = 1 - b1^step and bc2 = 1 - b2^step are computed by the caller. Hyper-parameters are
 * doubles, as the Python floats of the reference are; each is rounded to fp32 where the
 * reference's tensor op rounds it (1 - lr*wd, 1 - b1, lr/bc1, sqrt(bc2) are formed in double).
 * p, g, m, v share dtype w_dtype (state dtype = weight dtype, adamw.py:123-125);
 * mask is fp32. If wm != NULL the new effective masked weight is also written:
 * wm <- p * cast(hx*mask + (1-hx)*top2(mask)) (cols % 8 == 0 then; rows*cols = n).
 */
SF_API int sf_adamw_masked(void* p, const void* g, const float* mask, void* m, void* v, int w_dtype,
                    int64_t n, double lr, double beta1, double beta2, double eps, double weight_decay,
                    double decay, double bc1, double bc2, double adaptive_l1, void* wm, double hx,
                    int64_t cols, void* stream);

/*
 * The AMSGrad variant (amsgrad=True, legacy/adamw.py:126-128, 142-156): v_max <- max(v_max, v) after
 * v is updated, and the denominator is sqrt(v_max)/sqrt(bc2) + eps. v_max has dtype w_dtype.
 */
SF_API int sf_adamw_masked_amsgrad(void* p, const void* g, const float* mask, void* m, void* v, void* v_max,
                            int w_dtype, int64_t n, double lr, double beta1, double beta2, double eps,
                            double weight_decay, double decay, double bc1, double bc2, double adaptive_l1,
                            void* stream);

/*
 * The same AdamW step, followed in the same pass by the importance score of the UPDATED weight.
 *   replaces: AdamW.step legacy/adamw.py:65-176 followed by SparseLinear.update_mask's score
 *             refresh, legacy/sparse_modeling.py:1041-1088 (the training loop steps the optimizer,
 *             then update_mask scores the new weight: main.py's sparse step). One read of p, g,
 *             m, v, mask, H instead of the optimizer pass plus a score pass over W and H.
 * score[n] (fp32) <- metric(p_new as stored, H) (score = NULL: not written, only its statistics
 * are formed); norm[0..1] <- mean and population std + 1e-6 of score; scratch as for sf_hutch_score (scratch[0..1] hold sum and sum of squares on return).
 * metric is one of SF_METRIC_HESSIAN_OBD, _HESSIAN_RATIO, _MAGNITUDE, _HESSIAN; H (fp32) may be NULL
 * for _MAGNITUDE. hvp != NULL also folds this step's Hutchinson sample into H first
 * (H <- beta_h H + (1-beta_h) max(hvp*probe, 0), arguments as for sf_hutch_score; the reference
 * does it after backward and before the optimizer step, main.py's Hutchinson block); hvp = NULL
 * leaves H untouched. Results equal sf_hutch_score(score = NULL) + sf_adamw_masked +
 * sf_hutch_score(hvp = NULL), bit for bit in H, p, m, v and score.
 */
SF_API int sf_adamw_masked_score(void* p, const void* g, const float* mask, void* m, void* v, int w_dtype,
                          int64_t n, double lr, double beta1, double beta2, double eps, double weight_decay,
                          double decay, double bc1, double bc2, double adaptive_l1, const void* hvp,
                          const void* probe, int v_dtype, double beta_h, float* H, float* score, float* norm,
                          double* scratch, int metric, void* stream);

/*
 * Mask reductions for one layer (no mask update).
 *   replaces: mid_penalty legacy/utils.py:875-938, sparsity_penalty :941-1025,
 *             nm_2_4_tile_stats :1028-1234 (the per-layer sums; the caller combines layers).
 * stats as SF_MSTAT_* (FLIPS is left 0). cols % 4 == 0.
 */
SF_API int sf_mask_stats(const float* mask, double* stats, int64_t rows, int64_t cols, void* stream);

/*
 * Block-granular soft masks (hard_mask_type block_sparse16 / block_sparse32).
 *   replaces: the block branches of legacy/sparse_modeling.py: gate :1122-1157, _blockify_tensor
 *             :461-508, penalty :1395-1530, mask blockify :1600, hard projection :607-718.
 * The layer-wide decisions (quantile of the block scores, top-k blocks) are taken by the caller on
 * [rows/bs, cols/bs] arrays; these three entries are the passes over the layer itself.
 * sf_block_sums: sum[b], sumsq[b] (sumsq may be NULL) over every whole bs x bs block of x; with
 *   norm != NULL over (x - norm[0]) / norm[1] (the normalised score). bs = 16 or 32.
 * sf_block_mask_update: every element m of a whole block b moves to clamp((1-a) m + a G', 0, 1) with
 *   G' = gate[b], pulled by clamp(G' - pen (m - target[b]), 0, 1) when pen != 0 and pushed away from
 *   0.5 by the binarise factor; only new_sum[b], the block sums of the result, are written for
 *   whole blocks (sf_block_mask_apply re-writes them block-constant); elements beyond the whole
 *   blocks are updated in place with gate 1 and target 1.
 * sf_block_mask_apply: inside the whole blocks mask <- value[b] (value = NULL keeps the mask) and
 *   wm <- W * cast(hx * mask + (1 - hx) * keep[b]) (keep = 1 beyond the whole blocks); wm may be NULL.
 */
SF_API int sf_block_sums(const float* x, int64_t rows, int64_t cols, int bs, const float* norm, float* sum,
                  float* sumsq, void* stream);
SF_API int sf_block_mask_update(float* mask, int64_t rows, int64_t cols, int bs, const float* gate,
                         const float* target, double mask_lr, double pen, double binarize_decay,
                         float* new_sum, void* stream);
SF_API int sf_block_mask_apply(float* mask, const void* W, int w_dtype, void* wm, int64_t rows, int64_t cols,
                        int bs, const float* value, const uint8_t* keep, double hx, void* stream);

/*
 * mask_type / hard_mask_type 'structured' with a general N:M: every group of M consecutive entries
 * along the input dimension keeps its N largest (ties to the lower column).
 *   replaces: the structured gate legacy/sparse_modeling.py:1164-1185, beta mixing :1199-1225,
 *             'structured_topn' penalty :1532-1566 / 'mid' :1567-1570, binarize push :1575-1590,
 *             EMA :1593, flip count :1659-1661, _hard_mask_from_soft 'structured' :720-735 and the
 *             effective mask / weight*mask of forward :759-771, :74-81, for N:M other than 2:4
 *             (2:4 has sf_mask_update_nm24, which also writes the sparse tensor cores' metadata).
 * sf_mask_update_nm: the arithmetic of sf_mask_update_nm24 with topN-of-M in place of top2-of-4:
 *   s = (score - norm[0]) / norm[1]; G = sigmoid((s - tau_g)/(T + 1e-8)), tau_g the N-th largest s of
 *   the group (0/1 top-N indicator when structured_exact; the global *tau when tau != NULL); beta
 *   mixing, penalty (pulled from pen_mask when it is not NULL: the gate layer's mask in the GLU joint
 *   update, legacy/utils.py:363-479), binarise push, EMA, hard = topN(mask), wm <- W * cast(hx mask + (1-hx) hard)
 *   (optional). stats as SF_MSTAT_* (the TOP2 / BOT2 slots hold the sums of the kept / dropped
 *   entries). One thread per group. M in {2, 4, 8, 16, 32}, 1 <= N < M, cols % M == 0.
 * hard_view = SF_HARD_THRESHOLD makes the hard view (flip count, effective mask, kept / dropped sums)
 *   mask > 0.5, the 'unstructured' hard mask of :526-527; the groups then only shape beta mixing and
 *   the top-N pull, as in the reference.
 * sf_project_nm: hard 0/1 view of a soft mask (fp32 or bf16 in and out, row strides in elements).
 * sf_effective_weight_nm: wm <- W * cast(hx mask + (1 - hx) topN(mask)), or W * cast(mask) when
 *   finalized != 0 or hx >= 1 - 1e-6.
 */
SF_API int sf_mask_update_nm(const float* score, const float* norm, const float* tau, const float* pen_mask,
                      float* mask, const void* W, int w_dtype, void* wm, double* stats, int64_t rows, int64_t cols, int n_keep,
                      int m_group, double temperature, double mask_lr, double pen, int penalty_mode,
                      double beta_s, double binarize_decay, double hx, int structured_exact, int score_bf16,
                      int hard_view, void* stream);
SF_API int sf_project_nm(const void* soft, int in_dtype, int64_t ld_soft, void* hard, int out_dtype, int64_t ld_hard,
                  int64_t rows, int64_t cols, int n_keep, int m_group, void* stream);
SF_API int sf_effective_weight_nm(const void* W, int w_dtype, const float* mask, void* wm, int64_t rows,
                           int64_t cols, int n_keep, int m_group, double hx, int finalized, int hard_view,
                           void* stream);

/*
 * hard_mask_type 'block16': inside every 16 x 16 tile the keep_k entries with the largest soft-mask
 * value are kept (ties to the lower row-major position inside the tile).
 *   replaces: _hard_mask_from_soft 'block16' legacy/sparse_modeling.py:537-574, the 'block16'
 *             penalty :1298-1348, and for this mode the gate / EMA / flip count / effective mask
 *             of update_mask and forward (:1099-1162 unstructured gate, :1573-1663, :745-771).
 * sf_mask_update_tile16: sf_mask_update_nm24 with 16 x 16 tiles in place of groups of four:
 *   G = sigmoid((s - *tau)/(T + 1e-8)); penalty_mode 1: G = clamp(G - pen (mask - topk_tile(G)), 0, 1),
 *   2: G = clamp(G - pen (1 - 2 mask), 0, 1); binarise push; mask <- clamp((1-a) mask + a G, 0, 1);
 *   hard = topk_tile(mask); wm <- W * cast(hx mask + (1-hx) hard) (optional); stats as SF_MSTAT_*
 *   (the TOP2 / BOT2 slots hold the sums of the kept / dropped entries). One warp per tile, radix
 *   select of the k-th largest. rows and cols multiples of 16.
 * sf_project_tile16: hard view (fp32 0/1, optional) and / or masked weight of a soft mask.
 */
SF_API int sf_mask_update_tile16(const float* score, const float* norm, const float* tau, float* mask,
                          const void* W, int w_dtype, void* wm, double* stats, int64_t rows, int64_t cols,
                          int keep_k, double temperature, double mask_lr, double pen, int penalty_mode,
                          double binarize_decay, double hx, void* stream);
SF_API int sf_project_tile16(const float* soft, float* hard, const void* W, int w_dtype, void* wm, int64_t rows,
                      int64_t cols, int keep_k, double hx, void* stream);

/*
 * Logging summary of the soft masks.
 *   replaces: mask_stats legacy/utils.py:2069-2280 (the per-layer accumulation :2117-2154; the
 *             caller adds layers up, all-reduces and forms mean / std / entropy / fractions).
 * sf_mask_summary ADDS to out[0..12): count, sum m, sum m^2, sum of the binary entropy of
 *   clamp(m, eps, 1-eps) (clamp in fp32 as the reference's tensor op; fp32 logarithms, fp64 totals),
 *   counts m<0.5, m<0.1, m<0.01, m>0.9, m>0.99, m>0.5, sum of the m<0.5 entries, sum of the m>0.5
 *   entries. Zero `out` before the first layer.
 * sf_mask_sample_hist ADDS the histogram of mask[idx[0..take)) over `bins` equal bins of [0, 1]
 *   (torch.histc) to hist[0..bins): the reference's quantiles come from a random sample per layer.
 */
SF_API int sf_mask_summary(const float* mask, int64_t n, double eps, double* out, void* stream);
SF_API int sf_mask_sample_hist(const float* mask, const int64_t* idx, int64_t take, int bins, double* hist,
                        void* stream);

/*
 * Masked dense GEMMs (tcgen05 / TMEM / TMA, bf16 operands, fp32 accumulation).
 *   replaces: FusedMaskedLinearSTE.forward matmul, legacy/sparse_modeling.py:83-87,
 *             and .backward :105-129.
 * Operands are row-major 2-D; T = tokens. wm is the pre-masked weight [out, in].
 *   fwd  : y[T,out]  = alpha * x[T,in] . wm[out,in]^T  (+ bias[out])
 *   dgrad: dx[T,in]  = dy[T,out] . wm[out,in]
 *   wgrad: dw[out,in]= dy[T,out]^T . x[T,in]                      (no mask: STE)
 * dtype: SF_BF16 (tensor cores) or SF_F32 (fp32 FMA path, used for fp32 parity cases).
 * status (optional, device int32[4]): set non-zero if a bounded device-side wait ran
 * out; the output is then undefined. in, out, T multiples of 8; 16-byte aligned.
 */
SF_API int sf_masked_gemm_fwd(const void* x, const void* wm, const void* bias, void* y, int64_t T,
                       int64_t in, int64_t out, float alpha, int dtype, int32_t* status,
                       void* stream);
/*
 * Forward product with the low-rank bypass (SLoRB) inside the same launch:
 *   y[T,out] = x[T,in] . wm[out,in]^T + z[T,rank] . sw[out,rank]^T (+ bias[out])
 *   replaces: `out += (x x_proj^T) SLoRB_Weight^T` after the masked product,
 *             legacy/sparse_modeling.py:790-794, with z = x x_proj^T from sf_masked_gemm_fwd.
 * The K loop runs on over the second operand pair into the same accumulator, so the bypass costs
 * rank / in of the main product's time and no pass over y. bf16 only; more than 128 rows; rank a
 * multiple of 8 (a last K block that is not full is zero-filled by the loads).
 */
SF_API int sf_masked_gemm_fwd_lowrank(const void* x, const void* wm, const void* z, const void* sw,
                               const void* bias, void* y, int64_t T, int64_t in, int64_t out,
                               int64_t rank, int dtype, int32_t* status, void* stream);
SF_API int sf_masked_gemm_dgrad(const void* dy, const void* wm, void* dx, int64_t T, int64_t in,
                         int64_t out, int dtype, int32_t* status, void* stream);
SF_API int sf_masked_gemm_wgrad(const void* dy, const void* x, void* dw, int64_t T, int64_t in,
                         int64_t out, int dtype, int32_t* status, void* stream);

/*
 * Per-stream setting of the bf16 tensor-core products above (and of the sharded variants below): an
 * upper bound on the thread blocks of one launch on that stream (0 = all SMs, and forgets the stream),
 * so that two products on two streams can share the chip. No counterpart in the reference, whose
 * products are cuBLAS calls.
 */
SF_API int sf_masked_gemm_configure_stream(void* stream, int max_ctas);

/*
 * Bias gradient: db[out] = sum_t dy[t, out].
 *   replaces: grad_out_2d.sum(dim=0), legacy/sparse_modeling.py:127-129.
 * db is fp32 and is overwritten.
 */
SF_API int sf_bias_grad(const void* dy, int dtype, float* db, int64_t T, int64_t out, void* stream);

/*
 * Distillation KL loss over the vocabulary, one sweep of both logit tensors per direction.
 *   replaces: Distill_Model.kl_loss, legacy/sparse_modeling.py:1749-1828 (per chunk: clamp to
 *             +-max_logit, divide by the temperature, two log_softmax, exp, multiply, sum).
 * sf_kl_div_fwd: row_kl[r] = sum_v softmax(b)_v (log_softmax(b)_v - log_softmax(a)_v) with
 *   a = clamp(student[r], +-max_logit) / temperature, b likewise from teacher; lse[2r], lse[2r+1]
 *   = logsumexp of a and of b (kept for the backward pass). The caller sums the rows chunk by
 *   chunk (dropping chunks whose sum is not finite, :1802-1821) and scales by temperature^2 / rows.
 * sf_kl_div_bwd: grad[r, v] = row_scale[r] * (softmax(a)_v - softmax(b)_v) / temperature where
 *   |student[r, v]| < max_logit, else 0 (the gradient autograd gives the student logits; the
 *   teacher gets none). row_scale[r] = upstream gradient * temperature^2 / rows, 0 for dropped rows.
 * student, teacher, grad: [rows, vocab] of `dtype` (SF_F32 / SF_BF16), vocab % 8 == 0.
 */
SF_API int sf_kl_div_fwd(const void* student, const void* teacher, int dtype, int64_t rows, int64_t vocab,
                  double temperature, double max_logit, float* row_kl, float* lse, void* stream);
SF_API int sf_kl_div_bwd(const void* student, const void* teacher, int dtype, const float* lse,
                  const float* row_scale, int64_t rows, int64_t vocab, double temperature, double max_logit,
                  void* grad, void* stream);

/*
 * Row-sharded layer: the two products whose result has to cross GPUs, with the exchange done by
 * the GEMM epilogue itself (plain stores into the other GPUs' memory over NVLink) instead of a
 * collective that re-reads the result afterwards.
 *   replaces: the all-gather of the layer output and the reduce-scatter of the input gradient that
 *             FSDP / tensor-parallel wrappers run around a split layer (the reference wraps the
 *             model in FSDP, legacy/main_llama.py:603-621, and all-reduces through DDP otherwise).
 * sf_masked_gemm_fwd_allgather: this rank holds rows [col_offset, col_offset + out_local) of the
 *   weight; y_all[0..n_dest) are the FULL outputs [T, out_total] of every GPU (its own first or
 *   anywhere), and each tile of this rank's columns is stored into all of them.
 * sf_masked_gemm_dgrad_reducescatter: rank c owns token rows [c*T/n, (c+1)*T/n) of dX; slots[c] is
 *   the slot [T/n, in] that rank c keeps for THIS rank's partial sums (`rank` = this rank's index:
 *   the tiles are walked owner by owner in turn, starting after it). After all ranks finished
 *   (a barrier the caller provides), the owner adds its n slots with sf_reduce_slots.
 * sf_masked_gemm_fwd_multicast: the same all-gather through an NVSwitch multicast object: y_mc is
 *   the multicast address of the full output [T, out_total] (one buffer at the same offset on every
 *   GPU, all bound to one multicast object, e.g. torch symmetric memory's multicast_ptr); each
 *   16-byte piece leaves this GPU once (multimem.st) and the switch writes it into every GPU's
 *   copy, this GPU's included, so the traffic is 1/(n-1) of the per-destination stores.
 * All need T > 128 and bf16. Host arrays y_all / slots hold device pointers; peer pointers come from
 * sf_peer_open. No call waits on another GPU: ordering between ranks is the caller's barrier.
 */
SF_API int sf_masked_gemm_fwd_allgather(const void* x, const void* wm, const void* bias, void* const* y_all,
                                 int n_dest, int64_t T, int64_t in, int64_t out_local, int64_t out_total,
                                 int64_t col_offset, float alpha, int dtype, int32_t* status, void* stream);
SF_API int sf_masked_gemm_fwd_multicast(const void* x, const void* wm, const void* bias, void* y_mc, int64_t T,
                                 int64_t in, int64_t out_local, int64_t out_total, int64_t col_offset,
                                 float alpha, int dtype, int32_t* status, void* stream);
SF_API int sf_masked_gemm_dgrad_reducescatter(const void* dy, const void* wm, void* const* slots, int n_ranks,
                                       int rank, int64_t T, int64_t in, int64_t out_local, int dtype,
                                       int32_t* status, void* stream);
/* out[n] <- sum over g of slots[g*n .. g*n + n), fp32 accumulation in slot order. */
SF_API int sf_reduce_slots(const void* slots, void* out, int64_t n_slots, int64_t n, int dtype, void* stream);

/*
 * Owner-side sum of the partial input gradients through an NVSwitch multicast address:
 *   out[i] = sum over the GPUs bound to the multicast object of their copy of mc_src[i], i < n
 * (multimem.ld_reduce, fp32 accumulation in the switch, bf16, n a multiple of 8). Every rank writes
 * its whole partial [T, in] into its own symmetric buffer with the plain sf_masked_gemm_dgrad; after a
 * rank barrier each owner calls this on the multicast address of ITS rows: it receives 1/N of what the
 * store-based scatter (sf_masked_gemm_dgrad_reducescatter + sf_reduce_slots) lands on it, the product
 * runs at its local speed, and the transfer can run beside other work (max_ctas thread blocks, 0 = 64).
 * The order in which the switch adds the copies is not specified (fp32 accumulation, one rounding).
 *   replaces: the reduce-scatter of FSDP / tensor-parallel backward, legacy/main_llama.py:603-621.
 */
SF_API int sf_multimem_reduce(const void* mc_src, void* out, int64_t n, int dtype, int max_ctas, void* stream);

/*
 * Sharing a device buffer with the other processes of one node (one process per GPU) through CUDA
 * IPC. sf_peer_export fills `handle` (sf_peer_handle_bytes() bytes) and the offset of `ptr` inside
 * its allocation; the peer process passes both to sf_peer_open and gets a pointer valid on its own
 * device, to be released with sf_peer_close(base). The buffer must come from cudaMalloc (PyTorch's
 * default caching allocator does). No counterpart in the reference, which leaves this to NCCL.
 */
/*
 * Self-test of the device-side wait limit. Every mbarrier wait in the tensor-core kernels is
 * bounded (about two seconds); when one runs out the kernel stores a code in the caller's status
 * word, every role leaves through the common teardown, and the context stays usable. This entry
 * launches a one-block kernel that waits, with the same routine and a limit of `limit_ms`
 * milliseconds, on a barrier nobody arrives at: afterwards *status == 99. No counterpart in the
 * reference (its failure handling is host-side, legacy/main_llama.py:2075-2108).
 */
SF_API int sf_selftest_bounded_wait(double limit_ms, int32_t* status, void* stream);

/*
 * Issue-rate probe of the tensor cores (no counterpart in the reference): `ctas` thread blocks each
 * issue `iters` tcgen05.mma of shape 128 x n x 16 (bf16, fp32 accumulation) back to back, the A
 * operand read from shared memory (a_from_tmem = 0) or from tensor memory (1), and wait for them with a
 * bounded wait; cycles[0] (device, one int64) receives the slowest block's SM cycles for the batch, so
 * cycles[0] / iters is the cost of one MMA at that width. It is the measurement behind the choice to run
 * block-sparse-16 products on the dense tiles: a 16-wide MMA costs as many cycles as a 64-wide one.
 */
SF_API int sf_selftest_mma_issue_rate(int n, int a_from_tmem, int iters, int ctas, long long* cycles,
                                      int32_t* status, void* stream);

SF_API int sf_peer_handle_bytes(void);
SF_API int sf_peer_export(const void* ptr, void* handle, int64_t* offset);
SF_API int sf_peer_open(const void* handle, int64_t offset, void** base, void** ptr);
SF_API int sf_peer_close(void* base);

/*
 * Hard-2:4 compressed weights.
 *   replaces: the finalisation bake-in mask.copy_(hard); weight.mul_(mask),
 *             legacy/main_llama.py:2552-2563, and optimize_sparse_model_for_inference,
 *             legacy/eval_wiki_ppl.py:548-651 (the reference keeps the zeros dense; it has
 *             no compressed format).
 * values[out, in/2] (bf16): the two kept elements of each group of 4, in column order.
 * meta as in sf_mask_update_nm24. The kept set is top2 of `soft` (fp32, e.g. |W| or the
 * soft mask) with ties to the lower index.
 */
SF_API int sf_sparse24_compress(const void* W, const float* soft, void* values, uint8_t* meta,
                         int64_t out, int64_t in, void* stream);
/* Inverse of sf_sparse24_compress: dense[out,in] = W * hard (bf16). */
SF_API int sf_sparse24_decompress(const void* values, const uint8_t* meta, void* dense, int64_t out,
                           int64_t in, void* stream);

/* Bytes of the tensor-core ordered metadata buffer sf_sparse24_pack_meta writes. */
SF_API int64_t sf_sparse24_meta_tc_bytes(int64_t out, int64_t in);
/* Reorders logical metadata into the order the sparse tensor-core GEMM loads. */
SF_API int sf_sparse24_pack_meta(const uint8_t* meta, uint8_t* meta_tc, int64_t out, int64_t in,
                          void* stream);
/*
 * y[T,out] = x[T,in] . decompress(values, meta)^T  (+ bias) on the sparse tensor cores
 * (tcgen05.mma.sp, kind::f16). Same semantics as sf_masked_gemm_fwd with a binary 2:4
 * mask (legacy/sparse_modeling.py:72-93 after finalisation).
 */
SF_API int sf_sparse24_gemm(const void* x, const void* values, const uint8_t* meta_tc, const void* bias,
                     void* y, int64_t T, int64_t in, int64_t out, int32_t* status, void* stream);

/*
 * The same product for T <= 128 activation rows with the K range of each 128-row weight tile split
 * over several CTAs, so that a weight matrix with few tiles is streamed by all SMs (a 4096-row
 * matrix has 32 tiles for 148 SMs). Each K range stores its fp32 partial sums in `workspace`
 * (sf_sparse24_splitk_workspace_bytes(T, out) bytes, its first 64 KiB ZERO on first use: they hold
 * the tiles' arrival tickets, which every call leaves at zero again, so the workspace serves the next call
 * on the same stream). The last range to arrive adds the partial sums in K order, so the result
 * does not depend on timing; it agrees with sf_sparse24_gemm to fp32 rounding before the bf16
 * store. splits = 0 picks the factor; T > 128 ignores the workspace and runs sf_sparse24_gemm.
 * No counterpart in the reference (dense semantics as sf_sparse24_gemm).
 */
SF_API int64_t sf_sparse24_splitk_workspace_bytes(int64_t T, int64_t out);
SF_API int sf_sparse24_gemm_splitk(const void* x, const void* values, const uint8_t* meta_tc, const void* bias,
                            void* y, int64_t T, int64_t in, int64_t out, void* workspace,
                            int64_t workspace_bytes, int splits, int32_t* status, void* stream);

/*
 * Block-sparse-16 (block-CSR) weights.
 *   replaces: convert_to_block_sparse, legacy/triton_block_sparse.py:46-103 (same layout:
 *             blocks[nnz,16,16], row_ptr[out/16+1] int32, col_idx[nnz] int32; a block is
 *             kept iff sum|w*mask| > 0), built on the device instead of a Python loop.
 * Call with blocks == NULL to count: row_ptr is filled and *nnz_out (device int32) is set;
 * then call again with blocks/col_idx sized for nnz.
 */
SF_API int sf_bsr16_build(const void* W, const void* mask, int dtype, int mask_dtype, void* blocks,
                   int32_t* row_ptr, int32_t* col_idx, int32_t* nnz_out, int64_t out, int64_t in,
                   void* stream);
/* Scatters the kept blocks into a dense row-major [out,in] matrix (zeros elsewhere); the
 * device-side counterpart of the rebuild loop in BlockSparseLinear._torch_forward,
 * legacy/triton_block_sparse.py:435-462. */
SF_API int sf_bsr16_to_dense(const void* blocks, const int32_t* row_ptr, const int32_t* col_idx, void* dense,
                             int64_t in, int64_t out, int dtype, void* stream);
/*
 * Block-sparse-16 products.
 *   replaces: block_sparse_matmul_v2_kernel, legacy/triton_block_sparse.py:224-284 (fwd);
 *             dgrad / wgrad have no reference kernel: they are the dense STE backward of
 *             legacy/sparse_modeling.py:105-125 restricted to the kept blocks.
 *   fwd  : y[T,out]  = x[T,in] . Wbsr^T (+ bias)
 *   dgrad: dx[T,in]  = dy[T,out] . Wbsr
 *   wgrad: dblocks[nnz,16,16] = (dy^T . x) at the kept blocks
 * workspace: out*in elements of `dtype`, caller-owned, overwritten (the products run on the
 * dense tensor-core tiles through it). status as in sf_masked_gemm_fwd.
 */
SF_API int sf_bsr16_fwd(const void* x, const void* blocks, const int32_t* row_ptr, const int32_t* col_idx,
                        const void* bias, void* y, void* workspace, int64_t T, int64_t in, int64_t out,
                        int dtype, int32_t* status, void* stream);
SF_API int sf_bsr16_dgrad(const void* dy, const void* blocks, const int32_t* row_ptr, const int32_t* col_idx,
                          void* dx, void* workspace, int64_t T, int64_t in, int64_t out, int dtype,
                          int32_t* status, void* stream);
SF_API int sf_bsr16_wgrad(const void* dy, const void* x, const int32_t* row_ptr, const int32_t* col_idx,
                          void* dblocks, void* workspace, int64_t T, int64_t in, int64_t out, int dtype,
                          int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPARSEFORGE_B200_H */
