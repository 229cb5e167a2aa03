/* TEST INFRASTRUCTURE - not a product path.
 *
 * CPU restatement of the arithmetic of btb's decode hot path, used only as the checker by the tests, the smoke
 * entry and the benchmark's CPU-baseline leg. The shipped library never links or calls anything declared here.
 *
 * Two families of functions:
 *   orc_*          the card path's arithmetic (native/cuda/btb_kernels.cu of the reference): bf16 activations,
 *                  one warp a row, 32 lane chains of 8-element chunks, xor butterfly, bf16 outputs.
 *   btb_*          the CPU tier's C-ABI (native/src/lib.rs of the reference), same names and argument meaning:
 *                  f32 activations, 16 lane sums a row (column c to lane c mod 16), pairwise fold. This is both the
 *                  oracle of the expert GEMVs and the timed CPU baseline (AVX-512 when the host has it; the scalar
 *                  path writes the same bits).
 *
 * Parity pins: the widen functions are checked bit for bit against the reference's Python codecs (fixtures under
 * tests/golden made by tests/golden/make_golden.py), and the CPU-tier model step built from these functions is
 * checked against the reference's banked receipts for its tiny Qwen3 fixture.
 */
#ifndef BTB_ORACLE_H
#define BTB_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* error codes, native/src/lib.rs:17-33 */
#define BTB_OK 0
#define BTB_ERR_NULL (-1)
#define BTB_ERR_DOMAIN (-6)

/* ---- widens (packed -> bf16 bits / f32) ---------------------------------------------------------------- */

/* pack12, btb/pack12.py:70-97 and native/src/gemv.rs:737-793: weight i = (table[code_i] << 8) | lo[i], escapes
 * (ascending esc_idx) override the high byte. out: n bf16 bit patterns. */
int orc_widen_p12(const uint8_t* lo, const uint8_t* hi4, const uint8_t* table, const int32_t* esc_idx,
                  const uint8_t* esc_val, size_t n_esc, size_t n, uint16_t* out);
/* MXFP4, btb/mxfp4.py:102-124 and native/src/gemv.rs:1038-1062: fp4(code) * 2^(s-127), one exact multiply. */
int orc_widen_mxfp4(const uint8_t* blocks, const uint8_t* scales, size_t rows, size_t cols, float* out);
/* FP8, btb/fp8.py:36-46,97-100 and native/src/gemv.rs:2996-3085: bf16_rne(e4m3 * scale_f32[r/bm][c/bn]). */
int orc_widen_fp8(const uint8_t* w, const float* scales, size_t rows, size_t cols, size_t sr, size_t sc,
                  uint16_t* out);

/* ---- card-path arithmetic ------------------------------------------------------------------------------ */

/* native/cuda/btb_kernels.cu:89-142: y[m][r] = bf16(sum), lane l takes chunks l, l+32, .. of 8 in order. */
int orc_gemv_card_bf16(const uint16_t* w, const uint16_t* x, uint16_t* y, int M, int R, int C);
/* native/cuda/btb_kernels.cu:171-209: x[m][c] = bf16(bf16(silu(g)) * u) from gu [M, 2C] (gate then up). */
int orc_gemv_card_silu_bf16(const uint16_t* w, const uint16_t* gu, uint16_t* y, int M, int R, int C);
/* the same chains over packed weights widened on the fly (what the fused-widen kernels must equal) */
int orc_gemv_card_p12(const uint8_t* lo, const uint8_t* hi4, const uint8_t* table, const int32_t* esc_idx,
                      const uint8_t* esc_val, size_t n_esc, const uint16_t* x, uint16_t* y, int M, int R, int C);
int orc_gemv_card_fp8(const uint8_t* w, const float* scales, int sr, int sc, const uint16_t* x, uint16_t* y, int M,
                      int R, int C);
int orc_gemv_card_mxfp4(const uint8_t* blocks, const uint8_t* scales, const uint16_t* x, uint16_t* y, int M, int R,
                        int C);
/* native/cuda/btb_kernels.cu:470-480 */
int orc_silu_mul(const uint16_t* gu, uint16_t* m, int T, int I);
/* native/cuda/btb_kernels.cu:365-393; exact_rsqrt = 1 uses 1/sqrtf (the card's rsqrtf is an approximation) */
int orc_add_rmsnorm(uint16_t* h, const uint16_t* y, const uint16_t* w, float eps, uint16_t* x, int T, int H,
                    int centered);
/* native/cuda/btb_kernels.cu:261-327 (tbl may be null) */
int orc_norm_rope_kv(const uint16_t* qkv, const uint16_t* wq, const uint16_t* wk, float eps, const uint16_t* cos_t,
                     const uint16_t* sin_t, int n0, const int32_t* depth, uint16_t* K, uint16_t* V, uint16_t* qo,
                     int T, int Hq, int Hk, int D, long hs, long rs, int centered, const int32_t* tbl);
/* the decode attention's fold structure, native/cuda/btb_attn_flash.cuh:7-14,102-125: tiles of 64 keys, groups of
 * 8 tiles, log2-domain softmax, P rounded to bf16, states folded tile -> group -> row. Dot products and sums in
 * f32 in index order. sinks (f32 [Hq], may be null) joins one extra logit to the row's denominator. */
int orc_attn_decode(const uint16_t* q, const uint16_t* K, const uint16_t* V, uint16_t* out, int n0,
                    const int32_t* par, int T, int Hq, int Hk, int D, long hs, long rs, float scale, int win,
                    const int32_t* tbl, const float* sinks);
/* native/cuda/btb_kernels.cu:861-948 (mode 0: softmax -> top-k -> renormalise) and btb/engine/host.py:187-191
 * (mode 1: top-k of the logits -> softmax over the k). logits [T, ls] bf16 bits, or f32 when f32_logits. idx [T,k]
 * int32, w [T,k] bf16 bits. */
int orc_moe_route(const void* logits, int ls, int E, int k, int mode, int f32_logits, int32_t* idx, uint16_t* w, int T);
/* lowest-index argmax over bf16 logits rows, btb/engine/cuda.py:2237, native/src/sample.rs:57-67 */
int orc_argmax_bf16(const uint16_t* logits, int T, int V, int64_t* out);

/* the sampled pick, native/src/sample.rs:17-155,255-405 (whose kept set the card's kernels,
 * native/cuda/btb_kernels.cu:1865-2124, share): s = x * inv_t; top-k and top-p thresholds by radix select over exact
 * integer counts and 2^30 fixed-point masses; token = argmax(s + gumbel(key, i)) over the kept, lowest index first.
 * floors [R, 2] and margin [R] (the winner's lead in the race) may be null. */
int orc_sample_pick(const float* x, int R, int V, const uint64_t* keys, float inv_t, uint32_t top_k, float top_p,
                    uint32_t* out, uint32_t* floors, float* margin);
/* btb/sampling.py:22-31,59-61 `_mix` / `key_for`; :394-398 `_hash_uniform`; sample.rs:28-45 `fast_exp` */
uint64_t orc_sample_key(uint64_t seed, uint64_t pos, uint32_t salt);
float orc_sample_uniform(uint64_t key, uint32_t i);
float orc_sample_exp(float t);

/* ---- CPU tier C-ABI (reference names) ------------------------------------------------------------------ */

const char* btb_isa(void);
int32_t btb_gemv_bf16_rows(const uint16_t* w, size_t rows, size_t cols, const float* x, size_t b, float* y,
                           size_t threads);
int32_t btb_gemv_p12_rows(const uint8_t* lo, const uint8_t* hi4, const uint8_t* table, const int32_t* esc_idx,
                          const uint8_t* esc_val, size_t n_esc, size_t rows, size_t cols, const float* x, size_t b,
                          float* y, size_t threads);
int32_t btb_gemv_mxfp4_rows(const uint8_t* blocks, const uint8_t* scales, size_t rows, size_t cols, const float* x,
                            size_t b, float* y, size_t threads);
int32_t btb_gemv_fp8_rows(const uint8_t* w, const float* scales, size_t rows, size_t cols, size_t sr, size_t sc,
                          const float* x, size_t b, float* y, size_t threads);
/* f32 online-softmax GQA decode over a [hk, n, d] bf16 cache, native/src/attn.rs:400-439 (one part) */
int32_t btb_attn_decode_bf16(const float* q, const uint16_t* k, const uint16_t* v, size_t n, size_t hq, size_t hk,
                             size_t d, size_t k_head_stride, size_t v_head_stride, float scale, float* out,
                             size_t threads);
/* force the scalar path (1) or let the ISA probe decide (0): the two must write the same bits */
void orc_force_scalar(int on);

#ifdef __cplusplus
}
#endif
#endif
