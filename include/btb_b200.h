/* btb_b200 - the C-ABI of the sm_100a decode hot path.
 *
 * What binds here: btb launches its card kernels by name through a `Launcher`
 * (btb/engine/card_launch.py:428-440: launch(name, grid, block, args, stream, shared)) whose one implementation
 * loads native/cuda/btb_kernels.cu's fatbin with the CUDA driver API (btb/engine/native.py:1262-1316, 1405-1442).
 * Each function below replaces one kernel family of that fatbin; the reference kernel it stands in for is cited
 * beside it (file:line under native/cuda/ of btb). A `Launcher` built on these functions is a drop-in for the
 * reference's: same buffers, same argument meaning, same bits where the comment says so.
 *
 * Conventions (native/src/lib.rs:1-33 of btb, kept): every function returns 0 or a negative code, writes only
 * caller-owned buffers, never allocates and never synchronises. Pointers are DEVICE pointers unless the comment
 * says host. `stream` is a cudaStream_t (NULL = the legacy default stream); every call only enqueues and is legal
 * inside a stream capture. bf16 tensors are raw 16-bit patterns. Weight and activation pointers must be 16-byte
 * aligned. Device-side refusals (a cache slot past the capacity, a token id outside the table, a bounded wait that
 * ran out) are recorded in a status word read by btb_b200_status(); no kernel traps or spins without a limit.
 */
#ifndef BTB_B200_H
#define BTB_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BTB_B200_OK 0
#define BTB_B200_ERR_NULL (-1)     /* a required pointer is null (lib.rs:20) */
#define BTB_B200_ERR_DOMAIN (-6)   /* a zero, misaligned or unsupported dimension (lib.rs:27) */
#define BTB_B200_ERR_CUDA (-10)    /* the CUDA runtime refused the launch */
#define BTB_B200_ERR_TIMEOUT (-11) /* a bounded device-side wait ran out (status word only) */

int btb_b200_version(void);
int btb_b200_sm_count(void);
/* tunables: "ring_bytes", "seg_bytes", "x_smem_max", "ctas_per_sm", "evict_first", "pdl" (a mask: 1 the GEMV launches,
 * 2 the step's small kernels, 4 the MoE block's kernels start under programmatic dependent launch; default 5), "warps",
 * "balance", "solo", "moe_stream" (host string) */
int btb_b200_set_tuning(const char* key, int value);
/* reads the device status word into *code (host pointer) and clears it; synchronises the default stream's copy */
int btb_b200_status(int* code);

/* ---- GEMV family: y[M,R] = bf16(sum_c w[r][c] * x[m][c]), f32 accumulate, the card's chain order ---------------
 * M in {1,2,4,8,16,32}, C a multiple of 8. Row r of an M-row pass is the one-row step's row r to the bit. */

/* btb_gemv_bf16_m{M} (btb_kernels.cu:89-155). w [R,C] bf16, x [M,C] bf16, y [M,R] bf16. */
int btb_b200_gemv_bf16(const void* w, const void* x, void* y, int M, int R, int C, void* stream);
/* btb_gemv_mma_bf16 (native/cuda/btb_gemv_mma.cuh:123-315): the tensor-core matvec for passes of 1..32 rows - tcgen05.mma
 * with the accumulator in tensor memory, operand tiles by TMA tensor maps. One kernel for every pass width (x is read
 * as 32 rows, the rest zeros), so a row's bits do not depend on the width; its summation order is its own (as the
 * reference's is): it agrees with btb_b200_gemv_bf16 to rounding, not to the bit. workspace:
 * btb_b200_gemv_tc_workspace_bytes(R, C) bytes (0 for matrices of many rows), 16-byte aligned, for matrices of few
 * rows, which are cut over K: its first 1024 bytes are the tiles' arrival counters - ZERO before the first launch; a
 * launch leaves them at zero - and the rest the K ranges' partial sums; the CTA that arrives last on a tile adds them
 * in range order (the same sum every launch). One workspace serves every matrix of a stream. */
int btb_b200_gemv_tc_bf16(const void* w, const void* x, void* y, int M, int R, int C, void* workspace, void* stream);
/* btb_b200_gemv_tc_bf16 over pack12 weights read as stored (the parts of btb_b200_gemv_p12; `table` a HOST pointer to the
 * 16 high bytes): TMA brings a tile's stored parts, eight warps widen them in registers and write the bf16 operand tile
 * into shared memory in the MMA's swizzled layout - no widened copy in global memory, and the sums are
 * btb_b200_gemv_tc_bf16's over the widened matrix to the bit. C a multiple of 64; workspace as
 * btb_b200_gemv_tc_workspace_bytes(R, C). The widen of btb/pack12.py:71-97 in front of btb_gemv_mma_bf16
 * (btb_gemv_mma.cuh:123-315), which the reference runs over a widened copy (btb/engine/tiers.py:1198-1218). */
int btb_b200_gemv_tc_p12(const void* lo, const void* hi4, const void* table, const void* esc_idx, const void* esc_val,
                         const void* esc_row, const void* x, void* y, int M, int R, int C, void* workspace, void* stream);
size_t btb_b200_gemv_tc_workspace_bytes(int R, int C);
/* btb_gemv_mma_glu_silu (native/cuda/btb_gemv_mma.cuh:216-315): the gate/up form of the tensor-core matvec. w [2I, C]
 * (gate rows, then up rows), x [M, C]; m [M, I] = bf16(bf16(silu(g)) * u) over the matvec's bf16 outputs g, u at rows i
 * and I + i: btb_b200_gemv_tc_bf16 + btb_b200_silu_mul's bits without the [M, 2I] buffer. workspace as above
 * (btb_b200_gemv_tc_glu_workspace_bytes(I, C); 0 for matrices of many rows). */
int btb_b200_gemv_tc_glu_bf16(const void* w, const void* x, void* m, int M, int I, int C, void* workspace, void* stream);
size_t btb_b200_gemv_tc_glu_workspace_bytes(int I, int C);
/* btb_gemm_mma_bf16 (native/cuda/btb_gemm.cuh:154): the prefill GEMM y [T, R] = bf16(x [T, C] W^T) for a prompt chunk of
 * any T >= 1 on the same tcgen05 kernel - tiles of 128 weight rows by up to 256 x rows, every tile its whole K. An output
 * element is one accumulation over all of k in k order, so row t carries the bits btb_b200_gemv_tc_bf16 gives that row in
 * a pass of any width (the reference's rule for its GEMM and its tensor-core matvec, btb/engine/cuda.py:2827-2832). */
int btb_b200_gemm_tc_bf16(const void* w, const void* x, void* y, int T, int R, int C, void* stream);
/* btb_gemv_silu_bf16_m{M} (btb_kernels.cu:171-227): gu [M,2C] (gate then up), x = bf16(bf16(silu(g)) * u)
 * computed on the way in. M <= 8 and M*C*2 <= the x staging budget, else BTB_B200_ERR_DOMAIN (use
 * btb_b200_silu_mul + btb_b200_gemv_bf16: the same bits). */
int btb_b200_gemv_silu_bf16(const void* w, const void* gu, void* y, int M, int R, int C, void* stream);
/* pack12 weights (btb/pack12.py:48-97; the CPU form is btb_gemv_p12_rows, native/src/lib.rs:106-135) widened in
 * registers inside the GEMV; on a card the reference widens to a bf16 copy first (btb/engine/tiers.py:1198-1218)
 * and runs btb_gemv_bf16 - the output here is that output to the bit. lo u8[R*C], hi4 u8[R*C/2], table HOST
 * u8[16], esc_idx i32 / esc_val u8 the ascending escape list, esc_row i32[R+1] = for each row the first escape at
 * or past its start (btb_b200_p12_rows builds it; null when there are no escapes). C a multiple of 32. */
int btb_b200_gemv_p12(const void* lo, const void* hi4, const void* table, const void* esc_idx, const void* esc_val,
                      const void* esc_row, const void* x, void* y, int M, int R, int C, void* stream);
/* FP8 e4m3 weights + f32 [sr, sc] block scales (btb/fp8.py:36-100; the CPU form is btb_gemv_fp8_rows,
 * native/src/lib.rs:501-552): on a card the reference widens them to a bf16 copy at load (fp8.held) and runs
 * btb_gemv_bf16 - the output here is that output to the bit, each weight bf16(e4m3 * scale) made in registers.
 * C a multiple of 16, a scale block's columns a multiple of 8. */
int btb_b200_gemv_fp8(const void* w, const void* scales, int sr, int sc, const void* x, void* y, int M, int R, int C,
                      void* stream);
/* btb_gemv_silu over pack12 weights: the fold of btb_b200_gemv_silu_bf16 with the widen of btb_b200_gemv_p12. */
int btb_b200_gemv_silu_p12(const void* lo, const void* hi4, const void* table, const void* esc_idx,
                           const void* esc_val, const void* esc_row, const void* gu, void* y, int M, int R, int C,
                           void* stream);
/* btb_add_rmsnorm (btb_kernels.cu:365-393) folded into the GEMV that reads its output (btb_gemv_bf16_m{M}, :89-155):
 * every CTA computes x = rmsnorm(h_in + y_add) * norm_w on the way in (the same operations in the same order, so the
 * same bits as the two kernels), CTA 0 writes h_out = h_in + y_add. One launch instead of two, and the weight
 * copies are already in flight while the norm runs. y_add null: no add, h_out unused. h_out must not be h_in.
 * w alone: bf16 weights; hi4 not null: pack12 parts as btb_b200_gemv_p12 (table a HOST pointer). T live rows of the
 * M the pass is padded to (M <= 8); rows T..M-1 of y are computed over zeros. */
int btb_b200_gemv_norm(const void* w, const void* hi4, const void* table, const void* esc_idx, const void* esc_val,
                       const void* esc_row, const void* h_in, const void* y_add, const void* norm_w, float eps,
                       int centered, void* h_out, void* y, int T, int M, int R, int C, void* stream);
/* btb_b200_gemv_norm over FP8 weights: the prologue above, the widen of btb_b200_gemv_fp8 (scales f32 [sr, sc]) */
int btb_b200_gemv_norm_fp8(const void* w, const void* scales, int sr, int sc, const void* h_in, const void* y_add,
                           const void* norm_w, float eps, int centered, void* h_out, void* y, int T, int M, int R, int C,
                           void* stream);
/* the same with the SwiGLU of btb_silu_mul (btb_kernels.cu:481-484) in the epilogue: w is the merged gate/up block
 * [R = 2I, C] (gate rows, then up rows: btb/engine/cuda.py:1131-1164); a warp takes gate row p and up row p + I one
 * after the other and writes m[t][p] = bf16(bf16(silu(g)) * u) over the two bf16-rounded outputs - the bits
 * btb_gemv_bf16 + btb_silu_mul leave in m [M, I]. The [M, 2I] gate/up buffer is never written. */
int btb_b200_gemv_norm_swiglu(const void* w, const void* hi4, const void* table, const void* esc_idx,
                              const void* esc_val, const void* esc_row, const void* h_in, const void* y_add,
                              const void* norm_w, float eps, int centered, void* h_out, void* m_out, int T, int M, int R,
                              int C, void* stream);
/* esc_row[r] = lower_bound(esc_idx, r * C) for r in 0..R (the CPU kernel's per-row cursor, native/src/gemv.rs:720-735,
 * computed once at load instead of per call) */
int btb_b200_p12_rows(const void* esc_idx, int n_esc, int R, int C, void* esc_row, void* stream);
/* pack12's encoder (btb/pack12.py:48-68 `pack_bf16`) on the card, for a bf16 tensor [n] that already lies in device
 * memory; the parts are byte-identical to that encoder's. Four calls:
 *   _hist    counts the high bytes into hist (u32 [256], device; cleared by the call);
 *   _table   (host only, no device work) picks the table from the counts copied to the host: the 15 most frequent high
 *            bytes, by count descending and byte value ascending, unused slots 0; *n_codes = slots in use;
 *   _encode  writes lo [n] and hi4 [ceil(n/2)] (even element in the low nibble, an odd count's pad nibble 0) and leaves
 *            in tile_esc (i32 [btb_b200_p12_tiles(n) + 1]) each tile's first escape's position in the list, the total last;
 *   _escapes writes the escapes' ascending indices (i32) and high bytes from those offsets.
 * n at most 2^31 - 1 (escape indices are int32). */
size_t btb_b200_p12_tiles(long long n);
int btb_b200_p12_hist(const void* src, long long n, void* hist, void* stream);
int btb_b200_p12_table(const unsigned* hist_host, unsigned char* table16_host, int* n_codes);
int btb_b200_p12_encode(const void* src, long long n, const unsigned char* table16_host, int n_codes, void* lo, void* hi4,
                        void* tile_esc, void* stream);
int btb_b200_p12_escapes(const void* src, long long n, const unsigned char* table16_host, int n_codes,
                         const void* tile_off, void* esc_idx, void* esc_val, void* stream);

/* ---- the step's small kernels ------------------------------------------------------------------------------------ */

/* h[t,:] = table[ids[t],:] (btb/engine/cuda.py:2227-2232). ids int64 [T]. */
int btb_b200_embed(const void* table, const void* ids, void* h, int T, int H, int V, void* stream);
/* btb_add_rmsnorm (btb_kernels.cu:365-393): h += y (y may be null), x = bf16(h * rstd * w) or * (1 + w). */
int btb_b200_add_rmsnorm(void* h, const void* y, const void* w, float eps, void* x, int T, int H, int centered,
                         void* stream);
/* the same, and xf f32 [T, H] = x widened (the value the MoE block's router and experts read,
 * btb/engine/host.py:180-186): one launch for the norm and the widen */
int btb_b200_add_rmsnorm_wide(void* h, const void* y, const void* w, float eps, void* x, void* xf, int T, int H,
                              int centered, void* stream);
/* btb_silu_mul (btb_kernels.cu:481-484): m[T,I] = bf16(bf16(silu(g)) * u) over gu [T,2I]. */
int btb_b200_silu_mul(const void* gu, void* m, int T, int I, void* stream);
/* btb_norm_rope_kv{,_tbl}_d{64,128,256} (btb_kernels.cu:261-358): q/k RMSNorm (null weights: none), RoPE from bf16
 * tables [cap, D], K/V rows written to slot n0+t (through tbl when not null), q to [T,Hq,D]. cap: rows of the
 * tables and of the cache's logical range; a row past it is refused (status word). */
int btb_b200_norm_rope_kv(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t,
                          const void* sin_t, const void* n0p, const void* depth, void* K, void* V, void* q, int T,
                          int Hq, int Hk, int D, long long hs, long long rs, int centered, const void* tbl, int cap,
                          void* stream);
/* btb_norm_rope_kv_rows_d{64,128,256} (btb_kernels.cu:228-248, 258-327 ROWS): the rows layout - a pass's T rows as T
 * sequences a token each (a fork's rows, or a batch's). rw i32 on the card: [base, step, W, then (col, off, len) a row];
 * row t's keys are `len` cache rows from `off` (its prefix; forks share one) and then its own steps, step i at cache row
 * base + i * W + col. This pass's token stands at position len + step and its K/V go to that step's cache row; a row
 * with len < 0 is padding and computes nothing. cap: rows of the cache and of the tables. */
int btb_b200_norm_rope_kv_rows(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t,
                               const void* sin_t, const void* rw, void* K, void* V, void* q, int T, int Hq, int Hk, int D,
                               long long hs, long long rs, int centered, int cap, void* stream);
/* btb_attn_flash_d{64,128} (btb_attn_flash.cuh:372-675): decode / tree attention over the cache, split over groups
 * of 512 keys. part_m, part_l f32 [S,T,Hq], part_acc f32 [S,T,Hq,D], cnt i32 [T,Hk] zeroed once, S = ceil(cap/512).
 * sinks f32 [Hq] or null (gpt-oss: a logit joined to the softmax denominator, btb/engine/families/gpt_oss/sinks.py:
 * 203-229). Same tile/group/row folds as the reference; dot products in f32 on the SIMT cores (agrees to rounding). */
int btb_b200_attn_decode(const void* q, const void* K, const void* V, void* out, const void* n0p, const void* par,
                         int T, int Hq, int Hk, int D, long long hs, long long rs, float scale, void* part_m,
                         void* part_l, void* part_acc, void* cnt, int win, const void* tbl, const void* sinks, int cap,
                         void* stream);
/* btb_attn_flash_rows_d{64,128} (btb_attn_flash.cuh:286-290, 396-401): the rows layout's attention - row t reads its
 * own sequence's keys (rw as above) in logical order, the order a one-row step of that sequence alone reads them in, so
 * a row's bits are its own decode's whatever rows step beside it. Scratch as btb_b200_attn_decode's. */
int btb_b200_attn_decode_rows(const void* q, const void* K, const void* V, void* out, const void* rw, int T, int Hq,
                              int Hk, int D, long long hs, long long rs, float scale, void* part_m, void* part_l,
                              void* part_acc, void* cnt, int win, const void* sinks, int cap, void* stream);
/* the decode step's row (T = 1) in one launch: btb_norm_rope_kv_d* (btb_kernels.cu:261-358) and btb_attn_flash_d*
 * (btb_attn_flash.cuh:372-675) back to back in the reference. Every block rotates its kv head's queries itself; the
 * block whose key group holds slot n0 makes the new key and value, writes them to the cache and uses them from shared
 * memory. Arguments as the two functions above (qkv [1, (Hq+2Hk) D]; q [1, Hq, D] is still written); the cache, the
 * query buffer and `out` hold the bits the two launches would have left. D 64 or 128. cnt: i32 [Hq] here (under 4096
 * cached rows a kv head's query heads take a block each, and each counts its own groups in). */
int btb_b200_attn_step(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t,
                       const void* sin_t, const void* n0p, const void* depth, void* K, void* V, void* q, void* out,
                       int Hq, int Hk, int D, long long hs, long long rs, int centered, float scale, void* part_m,
                       void* part_l, void* part_acc, void* cnt, int win, const void* tbl, const void* sinks, int cap,
                       void* stream);
/* the same for B sequences decoded side by side (btb's batched greedy loop, btb/engine/generate.py:985-1046, over a
 * cache of B rows each at its own length, btb/engine/cache.py:334-337: the GEMVs run one pass of B rows, row b is
 * sequence b's token): qkv [B, (Hq+2Hk) D], n0p i32 [B] and depth i32 [B] (each sequence's length and 0), K / V
 * sequence 0's cache with `seq_stride` elements to the next sequence's, q [B, Hq, D], out [B, Hq D], partials
 * [B, S, Hq(, D)], cnt i32 [B, Hq]. Row b's bits are the one-sequence call's. */
int btb_b200_attn_step_batch(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t,
                             const void* sin_t, const void* n0p, const void* depth, void* K, void* V, void* q, void* out,
                             int B, long long seq_stride, int Hq, int Hk, int D, long long hs, long long rs,
                             int centered, float scale, void* part_m, void* part_l, void* part_acc, void* cnt, int win,
                             const void* sinks, int cap, void* stream);
/* btb_b200_attn_step and the output projection that reads its row (btb_gemv_bf16_m1 over o_proj, btb_kernels.cu:89-155)
 * as one cooperative launch: every CTA fills its ring with its rows of w_o [R, Hq D] first, the grid's CTAs share out
 * the attention's blocks, meet at one bounded grid barrier and multiply. att [1, Hq D] is still written; y [1, R] bf16.
 * bar: u32 [2] on the card, zero before the first launch, used by no other stream at the same time. The bits are the
 * two launches' bits. No row map. The device must hold the whole grid at once (one CTA an SM): the launch is refused
 * (ERR_CUDA) where it cannot. */
int btb_b200_attn_o_step(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t,
                         const void* sin_t, const void* n0p, const void* depth, void* K, void* V, void* q, void* att,
                         int Hq, int Hk, int D, long long hs, long long rs, int centered, float scale, void* part_m,
                         void* part_l, void* part_acc, void* cnt, int win, const void* sinks, int cap, const void* w_o,
                         void* y, int R, void* bar, void* stream);
size_t btb_b200_attn_scratch_floats(int S, int T, int Hq, int D);
/* the greedy pick: lowest-index argmax of each bf16 logits row (torch.argmax in btb/engine/cuda.py:2237; tie rule
 * native/src/sample.rs:57-67). scratch: btb_b200_argmax_scratch_bytes(T) bytes, 8-byte aligned, zeroed once.
 * out int64 [T]. */
int btb_b200_argmax_bf16(const void* logits, int T, int V, void* scratch, void* out, void* stream);
size_t btb_b200_argmax_scratch_bytes(int T);
/* The same pick with no scratch argument. This entry point has no counterpart in the reference. It is for callers that
 * cannot allocate device memory when they need the pick - a host whose device budget was fixed at start-up, or code
 * already inside a stream capture, where cudaMalloc is illegal - the scratch is an array built into the library
 * (a few hundred bytes on every device that loads it, held until exit). T at most 32 rows (BTB_B200_ERR_DOMAIN
 * beyond). It allocates nothing and frees nothing. The first call on each device looks the array's address up:
 * make that call before starting any stream capture. All calls share the one array: two calls whose kernels may
 * overlap on the device (different streams) race on it - keep them on one stream or order them yourself. */
int btb_b200_argmax_bf16_static(const void* logits, int T, int V, void* out, void* stream);
/* the sampled pick: btb_sample_keys / _max / _hist / _bin / _draw / _out (native/cuda/btb_kernels.cu:1865-2124) and
 * btb_sample_pick (native/src/sample.rs:385-405) as one launch - a cluster of 8 CTAs a row. logits [R, V] at stride
 * `ls`, bf16 (or f32 when f32_logits); fp f32 [2] ON THE CARD = {1 / temperature, top_p} (top_p >= 1 switches the
 * nucleus off); top_k 0 = off. The row's key is keys[r] (u64 on the card), or with keys null
 * key_for(seed, *n0p + depth[r], salt) (btb/sampling.py:57-61; seed u64 and n0p i32 on the card, depth i32 [R] or
 * null). out i64 [R] (or null). floors u32 [R, 2] or null: the top-k and top-p thresholds as ordered float bits.
 * packed u64 [R] or null: the winner as btb_sample_draw leaves it in `gbest` (ordered value << 32 | ~index). The kept
 * set is the reference's to the token; V is limited by a CTA's shared memory (an eighth of the row as f32: V <= ~360k). */
int btb_b200_sample_pick(const void* logits, int f32_logits, int R, int V, long long ls, const void* fp, int top_k,
                         const void* keys, const void* seed, const void* n0p, const void* depth, unsigned salt,
                         void* out, void* floors, void* packed, void* stream);
/* btb_sample_verify (native/cuda/btb_kernels.cu:2126-2359; host side btb/sampling.py:272-372 `Verify`): the pick of a
 * verify pass whose rows are tree nodes with drafted children - exact rejection sampling, the emitted token a draw from
 * the target at every node. logits [R, V] at stride ls (f32 when f32_logits, else bf16); q f32 [R, Vd] the drafter's
 * masses a node (unnormalised is fine); kids i32 [R, C] a node's children in draw order, -1 after the last, C <= 32;
 * hasq u32 [R] (0: the node's drafts are point masses - it draws from the target and accepts the child that equals the
 * draw); keys u64 [R]; fp f32 [2] = [1/T, top_p] on the card. out u32 [R] = (accepted slot + 1) << 24 | token, slot 0
 * when no child was accepted. One launch: the thresholds and the point-mass race on a cluster of 8 CTAs a row, the
 * trials' floating-point sums on the cluster's first CTA in the reference's order (1024 threads striding the row, warps
 * folded by halving strides, the warps' sums added in order). */
int btb_b200_sample_verify(const void* logits, int f32_logits, int R, int V, long long ls, const void* q, int Vd,
                           const void* kids, int C, const void* hasq, const void* keys, int top_k, const void* fp,
                           void* out, void* stream);
/* btb_sample_out (native/cuda/btb_kernels.cu:2110-2114): out u32 [R] = the token of each packed winner */
int btb_b200_sample_out(const void* packed, void* out, int R, void* stream);
/* btb_sample_keys (native/cuda/btb_kernels.cu:2116-2124): keys u32 [2] = key_for(seed u32 [2] (lo, hi), pos i32 [1],
 * salt) as (lo, hi), for callers that keep the reference's separate key buffer */
int btb_b200_sample_keys(const void* seed, const void* pos, unsigned salt, void* keys, void* stream);
/* the tree commit (btb/engine/cuda.py:3535-3575 `ad`): a verify pass's accepted path gathered in place - node path[j]'s
 * row (slot n0 + path[j]) moves to slot n0 + j in every layer's K and V. K, V: layer 0's arenas, `layer_stride`
 * elements to the next layer's, a row `row_el` elements at stride `rs`. path i32 [len] on the card, parents first
 * (path[j] >= j; else refused through the status word). n0 is not advanced here (btb_b200_publish does). */
int btb_b200_kv_commit(void* K, void* V, long long layer_stride, int layers, const void* n0p, const void* path, int len,
                       int row_el, long long rs, const void* tbl, int cap, void* stream);
/* ---- drafting, host side (no device work, no stream) ----------------------------------------------------------------
 * btb's n-gram proposer (btb/draft.py:8-113 `NGramProposer`): for each order n in [n_min, n_max] every n-gram of the
 * text remembers its followers, how often and where last. _new returns a handle (null: orders not served), _extend
 * appends tokens, _free releases. */
void* btb_b200_ngram_new(int n_max, int n_min, int followers);
void btb_b200_ngram_free(void* proposer);
int btb_b200_ngram_extend(void* proposer, const long long* toks, int n);
int btb_b200_ngram_length(void* proposer);
/* `propose_chains(v)` (btb/draft.py:76-97): continuations of the text's tail of up to v tokens, longest order first, most
 * frequent then most recent follower first, a chain that is a prefix of an earlier one dropped. Chain c is
 * toks[offs[c] .. offs[c + 1]) found at order[c]; toks holds max_chains * v, offs max_chains + 1, order max_chains. */
int btb_b200_ngram_chains(void* proposer, int v, int max_chains, int* toks, int* offs, int* order, int* n_chains);
/* `_chains_tree` (btb/engine/generate.py:94-117): chains merged by shared prefix into a tree of at most `budget` guesses;
 * node 0 is the root, node j > 0 carries guesses[j - 1]; parents and depth hold budget + 1, parents first. */
int btb_b200_chains_tree(const int* toks, const int* offs, int n_chains, int budget, int* guesses, int* parents, int* depth,
                         int* n_guesses);
/* btb_b200_ngram_chains then btb_b200_chains_tree in one call */
int btb_b200_ngram_tree(void* proposer, int v, int budget, int* guesses, int* parents, int* depth, int* n_guesses);
/* the accept walk of a verify pass (btb/engine/generate.py:765-795): from the root, the child whose guess is its parent's
 * own pick, while there is one. picks i64 [n_nodes], guesses [n_nodes - 1], parents [n_nodes]; path holds n_nodes. */
int btb_b200_tree_walk(const long long* picks, const int* guesses, const int* parents, int n_nodes, int* path, int* n_path);

/* btb_publish (btb_kernels.cu:455-465): n0 += advance, then token, device clock (ns) and length to pinned host memory,
 * the length last behind a system fence. out_* null: only the advance. */
int btb_b200_publish(void* n0, const void* ids, void* out_tok, void* out_n0, void* out_ts, int advance, void* stream);

/* ---- the MoE block ------------------------------------------------------------------------------------------------
 * btb_moe_route (btb_kernels.cu:861-948) and the host routers it mirrors. mode 0: f32 softmax over the E logits ->
 * top-k by (p desc, index asc) -> p / sum(top k) (btb/engine/families/qwen4/router.py:42-50); mode 1: top-k of the
 * logits -> softmax over the k (gpt-oss, btb/engine/host.py:187-191). logits [T, ls] bf16, or f32 when f32_logits;
 * idx i32 [T,k], w bf16 [T,k]. */
int btb_b200_moe_route(const void* logits, int ls, int E, int k, int mode, int f32_logits, void* idx, void* w, int T,
                       void* stream);
/* the router's matvec (btb_gemv_lane16_f32_m*, btb_kernels.cu:1635-1700; the host's _Router, btb/engine/host.py:175-191)
 * and btb_moe_route's picks as one launch: a cluster of 8 CTAs a row, the logits handed to the leader through
 * distributed shared memory. w bf16 [E, H], x f32 [T, H], logits f32 [T, E] or null (written when given), idx i32 [T, k],
 * wout bf16 [T, k]. The logits and the picks are the two calls' to the bit. H a multiple of 8, E <= 1024. */
int btb_b200_moe_router(const void* w, const void* x, void* logits, int E, int H, int k, int mode, void* idx, void* wout,
                        int T, void* stream);
/* btb_b200_add_rmsnorm_wide and btb_b200_moe_router as one launch: the block's residual add, RMSNorm and widen
 * (btb_add_rmsnorm, btb_kernels.cu:365-393; the row widened to f32 for the host-order experts, btb/engine/host.py:180-186)
 * in the router launch's prologue. h_in, y_add (may be null), norm_w bf16; h_out the new residual (required with y_add, never
 * h_in's buffer); xf_out f32 [T, H] the widened normed row (what the experts read), x_out bf16 [T, H] or null. The same
 * operations in the same order as the two launches: the same bits. */
int btb_b200_moe_router_norm(const void* w, const void* h_in, const void* y_add, const void* norm_w, float eps, int centered,
                             void* h_out, void* x_out, void* xf_out, void* logits, int E, int H, int k, int mode, void* idx,
                             void* wout, int T, void* stream);
/* btb_b200_moe_router_norm for routers of any size (no counterpart in the reference: its host issues the norm, the matvec
 * and btb_moe_route apart): a grid of CTAs a token over the whole card instead of one cluster; each takes a few experts'
 * rows, writes their logits to `logits` f32 [T, E] (required) and counts itself in at cnt i32 [T] (zero before the first
 * launch, left zero); the CTA that arrives last picks - no CTA waits for another. h_in null: no norm, x f32 [T, H] is read
 * from xf_out. The same bits as the separate launches. */
int btb_b200_moe_router_grid(const void* w, const void* h_in, const void* y_add, const void* norm_w, float eps, int centered,
                             void* h_out, void* x_out, void* xf_out, void* logits, void* cnt, int E, int H, int k, int mode,
                             void* idx, void* wout, int T, void* stream);
/* btb_gemv_lane16_f32_m{M} (btb_kernels.cu:1635-1682): the host's bf16 GEMV order on the card (16 lane sums a row,
 * column c to lane c mod 16, reduce16's fold: native/src/gemv.rs:46-58,85-123). w [R,C] bf16, x [M,C] f32, y [M,R]
 * f32; bit-equal to btb_gemv_bf16_rows. */
int btb_b200_gemv_lane16_f32(const void* w, const void* x, void* y, int M, int R, int C, void* stream);
/* btb_gemv_lane16_mx4_f32_m{M} (btb_kernels.cu:1684-1766): the same over MXFP4 as stored (blocks [R,C/32,16],
 * scales [R,C/32] e8m0); bit-equal to btb_gemv_mxfp4_rows (native/src/lib.rs:137-160). */
int btb_b200_gemv_lane16_mx4_f32(const void* blocks, const void* scales, const void* x, void* y, int M, int R, int C,
                                 void* stream);
/* the same over FP8 e4m3 + f32 [sr,sc] block scales, each weight bf16(e4m3 * scale); bit-equal to btb_gemv_fp8_rows
 * (native/src/lib.rs:501-552, gemv.rs:2996-3085). */
int btb_b200_gemv_lane16_fp8_f32(const void* w, const void* scales, int sr, int sc, const void* x, void* y, int M,
                                 int R, int C, void* stream);
/* `_Experts._one_row`'s grouped matvec (btb/engine/host.py:508-569; btb_gemv_*_group, native/src/lib.rs:86-104,
 * 162-243) with the picks read on the card: task i multiplies expert idx[i]'s [R,C] matrix (fmt 0 bf16, 1 MXFP4,
 * 2 FP8; w_stride/s_stride bytes between experts) with x row i / x_div; y f32 [n_tasks, R]. An index outside
 * [0, E) is refused (status word). Expert parallelism: `w` holds this rank's experts only, expert e being local expert
 * e / ep_size of rank e % ep_size; a task of another rank's expert writes a row of zeros (ep_size 1: everything). */
int btb_b200_moe_gemv(int fmt, const void* w, const void* scales, long long w_stride, long long s_stride, int sr,
                      int sc, const void* idx, int n_tasks, int E, const void* x, int x_div, void* y, int R, int C,
                      int ep_rank, int ep_size, void* stream);
/* the experts' middle (host.py:414-419): gu f32 [n,2I] to the row dtype (+ bias [E,2I] bf16 by idx), kind 0
 * silu(gate) * up over halves (host.py:439-441), kind 1 gpt-oss's clamped GLU over interleaved lanes
 * (host.py:444-450; btb/mxfp4_torch.py:146-153), every bf16 rounding of the torch ops kept; h f32 [n,I]. */
int btb_b200_moe_act(const void* gu, void* h, const void* bias, const void* idx, int n, int I, int kind, float alpha,
                     float limit, void* stream);
/* btb_b200_moe_act then btb_b200_moe_gemv as one launch: task i's x row is the gated activation of gu row i
 * (f32 [n_tasks, 2C]; kind, alpha, limit as btb_b200_moe_act; no bias), made while the expert's rows are on their
 * way. y f32 [n_tasks, R]. Shapes the streaming kernel does not take (C not a multiple of 32, unaligned rows) are
 * refused: use the two calls. */
int btb_b200_moe_gemv_act(int fmt, const void* w, const void* scales, long long w_stride, long long s_stride, int sr,
                          int sc, const void* idx, int n_tasks, int E, const void* gu, int kind, float alpha,
                          float limit, void* y, int R, int C, int ep_rank, int ep_size, void* stream);
/* the picked experts' GATE/UP matvecs with the gated activation (btb/engine/host.py:439-450) made on the way out: h f32
 * [n_tasks, R/2] row i = act(task i's [R] outputs), every bf16 rounding of the host's torch ops kept; the [n_tasks, R]
 * outputs are never written. kind 0 pairs gate row j with up row R/2 + j (silu(gate) * up), 1 pairs rows 2j and 2j + 1
 * (gpt-oss's clamped GLU with alpha, limit). btb_b200_moe_gemv followed by btb_b200_moe_act, one launch. No bias. Shapes
 * the streaming kernel takes, R a multiple of 8. */
int btb_b200_moe_gemv_glu(int fmt, const void* w, const void* scales, long long w_stride, long long s_stride, int sr, int sc,
                          const void* idx, int n_tasks, int E, const void* x, int x_div, void* h, int R, int C, int kind,
                          float alpha, float limit, int ep_rank, int ep_size, void* stream);
/* host.py:426-431,565-569: out_e = bf16(down_e) (+ bias [E,H]) * w_e, summed one bf16 add at a time in ascending
 * expert id from zero. dn f32 [T,k,H], y bf16 [T,H]. */
int btb_b200_moe_combine(const void* dn, const void* idx, const void* w, const void* bias, void* y, int T, int k, int H,
                         void* stream);
/* btb_b200_moe_combine (no bias) and the btb_b200_add_rmsnorm that reads its row, one launch: the ordered bf16 sum of
 * the k picks, h = bf16(h + sum), x = bf16(h * rstd * norm_w); xf (f32, may be null) = x widened; y (may be null)
 * receives the sum itself. The bits are the two launches'. */
int btb_b200_moe_combine_norm(const void* dn, const void* idx, const void* w, int k, void* h, const void* norm_w,
                              float eps, void* x, void* xf, void* y, int T, int H, int centered, void* stream);
/* x.float() (host.py:525): bf16 [n] -> f32 [n] */
int btb_b200_widen_f32(const void* x, void* y, int n, void* stream);

/* ---- one model over the GPUs of a box (one process a GPU): the exchange ---------------------------------------------
 * btb has no multi-GPU path (no counterpart in the reference); these serve `north_star`'s sharded configurations with the
 * one-GPU bits. Every linear is cut by OUTPUT rows, so ranks exchange finished bf16 elements, never partial sums. An
 * exchanged vector lives in every rank's memory as u32 WORDS [M, stride]: a word is the element's bf16 in its low half
 * and, in its high half, the low 16 bits of the hop's sequence number pass * per_pass + base. A producer stores each
 * finished element's word into every rank's copy (plain 4-byte stores to peer-mapped memory: atomic, no fence, no flag);
 * a consumer reads its local copy and takes a word once it carries the hop's mark (re-reading until then: about a second
 * at most, then BTB_B200_ERR_TIMEOUT in the status word, and the kernel goes on). `pass` is a device-side u32 count of
 * the passes made so far, advanced once a pass (btb_b200_xchg_pick or btb_b200_xchg_tick), so a captured graph replays
 * without new arguments; `base` numbers the hop within the pass (1 ..per_pass). */
typedef struct btb_b200_recv {
    const void* pass;  /* the pass count (device, u32) */
    unsigned per_pass; /* hops a pass makes */
    unsigned base;     /* this hop's number within the pass */
} btb_b200_recv;
typedef struct btb_b200_send {
    void* out[8]; /* every rank's copy of the full vector (u32 words), this rank's own included; peer-mapped, 16-byte aligned */
    int n;        /* ranks; 0: no exchange */
    int stride;   /* elements a row of the full vector holds */
    int offset;   /* where this rank's slice starts in a row */
    const void* pass;
    unsigned per_pass, base;
} btb_b200_send;
/* peer-mapped memory for one-process-a-GPU jobs (no counterpart in the reference). SET-UP calls: _alloc is cudaMalloc
 * (zeroed) and the others open and close CUDA IPC handles; none belongs in a decode loop or a stream capture. handle64:
 * 64 host bytes to hand to the other processes of the box (any channel), which _open them into pointers valid in their
 * own address space. */
int btb_b200_peer_alloc(size_t bytes, void** ptr);
int btb_b200_peer_free(void* ptr);
int btb_b200_peer_handle(void* ptr, unsigned char* handle64);
int btb_b200_peer_open(const unsigned char* handle64, void** ptr);
int btb_b200_peer_close(void* ptr);
/* btb_b200_gemv_bf16 with the exchange folded in: with `recv`, x is this rank's copy of an exchanged vector (words
 * [M, C]), its T live rows taken word by word on their way into shared memory, the padding rows read as zeros (M <= 8 and
 * M*C*2 within the x staging budget, else BTB_B200_ERR_DOMAIN: btb_b200_xchg_unpack first); with send->n > 0 the
 * outputs go, marked, to every rank's copy at [m][offset + r] (y may be null). */
int btb_b200_gemv_bf16_x(const void* w, const void* x, void* y, int T, int M, int R, int C, const btb_b200_recv* recv,
                         const btb_b200_send* send, void* stream);
/* btb_b200_gemv_norm (swiglu 0) / btb_b200_gemv_norm_swiglu (swiglu 1) over bf16 weights with the exchange folded in:
 * with `recv`, y_add is this rank's copy of an exchanged vector */
int btb_b200_gemv_norm_x(const void* w, const void* h_in, const void* y_add, const void* norm_w, float eps, int centered,
                         void* h_out, void* y, int T, int M, int R, int C, int swiglu, const btb_b200_recv* recv,
                         const btb_b200_send* send, void* stream);
/* btb_b200_attn_step / btb_b200_attn_decode in a model cut over ranks by kv head (this rank's Hq query and Hk kv heads):
 * the output rows go, marked, to every rank's copy of the full [T, stride] vector at [t][offset + head * D + d] */
int btb_b200_attn_step_x(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t, const void* sin_t,
                         const void* n0p, const void* depth, void* K, void* V, void* q, int Hq, int Hk, int D, long long hs,
                         long long rs, int centered, float scale, void* part_m, void* part_l, void* part_acc, void* cnt,
                         int win, const void* tbl, const void* sinks, int cap, const btb_b200_send* send, void* stream);
int btb_b200_attn_decode_x(const void* q, const void* K, const void* V, const void* n0p, const void* par, int T, int Hq,
                           int Hk, int D, long long hs, long long rs, float scale, void* part_m, void* part_l,
                           void* part_acc, void* cnt, int win, const void* tbl, const void* sinks, int cap,
                           const btb_b200_send* send, void* stream);
/* btb_b200_attn_step (send null or n 0; out the local row) or btb_b200_attn_step_x (send set; out may be null) with the
 * SMs the row leaves idle pulling up to the `l2_warm_kb` tunable of the next kernels' weights into L2 meanwhile - warm_a
 * first, then warm_b (device pointers and byte counts, 16-byte aligned; null or 0: none). The reference warms L2 ahead of
 * its tensor-core matvec with a kernel of its own (btb_l2_warm, native/cuda/btb_gemv_mma.cuh:317-357). */
int btb_b200_attn_step_w(const void* qkv, const void* wq, const void* wk, float eps, const void* cos_t, const void* sin_t,
                         const void* n0p, const void* depth, void* K, void* V, void* q, void* out, int Hq, int Hk, int D,
                         long long hs, long long rs, int centered, float scale, void* part_m, void* part_l, void* part_acc,
                         void* cnt, int win, const void* tbl, const void* sinks, int cap, const btb_b200_send* send,
                         const void* warm_a, long long bytes_a, const void* warm_b, long long bytes_b, void* stream);
/* (no counterpart in the reference) a finished local slice src bf16 [M, n] into every rank's copy, marked: for kernels
 * that do not send themselves. n, stride and offset multiples of 4. */
int btb_b200_xchg_send(const void* src, int M, int n, const btb_b200_send* send, void* stream);
/* (no counterpart in the reference) this rank's copy of an exchanged vector (words [M, C]) as plain bf16 dst [M, C] once
 * every word carries the hop's mark: for consumers that read plain vectors (wide passes), and where a wait on its own
 * is wanted. M: the rows to take (a pass's live rows - a producer may send none for its padding rows). C a multiple of 8. */
int btb_b200_xchg_unpack(const void* words, void* dst, int M, int C, const btb_b200_recv* recv, void* stream);
/* the greedy pick over a vocabulary cut by rows: local_idx i64 [T] is this rank's lowest-index argmax within its slice
 * logits [T, Vl] (btb_b200_argmax_bf16); every rank receives every rank's (value, v_offset + index) and takes the largest
 * value, the lowest index among equals - the one-GPU pick (btb/engine/cuda.py:2237). tables (host array of `ranks` device
 * pointers): rank p's table, u64 [ranks, 32, 2], zero at first. pick_pass: the picks' own pass count (device u32,
 * advanced here); body_pass (may be null): the layers' pass count, advanced by one at the end too. ids i64 [T]. phase 0:
 * the whole pick; 1: send only; 2: take and merge only (for ranks that share one GPU and take turns). T <= 32. */
int btb_b200_xchg_pick(const void* logits, int T, int Vl, int v_offset, const void* local_idx, int rank, int ranks,
                       void* const* tables, void* ids, void* pick_pass, void* body_pass, int phase, void* stream);
/* experts cut over ranks (expert e on rank e % ep_size): btb_b200_moe_gemv whose outputs for the experts this rank holds
 * go to every rank's copy of the [n_tasks, R] vector as marked words carrying bf16(output) - the rounding
 * btb_b200_moe_combine applies to a product first - and btb_b200_moe_combine reading such a copy. send->stride = R,
 * send->offset = 0. */
int btb_b200_moe_gemv_x(int fmt, const void* w, const void* scales, long long w_stride, long long s_stride, int sr, int sc,
                        const void* idx, int n_tasks, int E, const void* x, int x_div, int R, int C, int ep_rank, int ep_size,
                        const btb_b200_send* send, void* stream);
int btb_b200_moe_combine_x(const void* dn_words, const void* idx, const void* w, const void* bias, void* y, int T, int k,
                           int H, const btb_b200_recv* recv, void* stream);
/* a pass-count advance as a launch of its own (no counterpart in the reference) */
int btb_b200_xchg_tick(void* pass, void* stream);

/* ---- the whole step as one launch ---------------------------------------------------------------------------------
 * btb captures a decode step as a CUDA graph of ~330 kernel nodes (btb/engine/cuda.py:2101-2251 `_card_step_graph`
 * over `_card_body`, :1601-1837). btb_b200_step runs the same sequence - embed, every layer's kernels, the head, the
 * greedy pick, the publish (btb_kernels.cu:455-465) - as ONE persistent cooperative kernel that walks a program of
 * phases, its TMA rings prefetching the next GEMV's weights across the grid barriers. `args`: a HOST image of the
 * kernel's argument record and, through it, a DEVICE array of phase records (btb_b200/step.py builds both; their
 * sizes are btb_b200_step_args_bytes / btb_b200_step_op_bytes). M: the pass width (1 or 2), D: head dim (128),
 * G: query heads a kv head (2, 4, 8). The barrier counter and abort flag the record points at must be zero at launch.
 * Bit-identical to the separate launches above. */
int btb_b200_step(const void* args, int M, int D, int G, void* stream);
size_t btb_b200_step_op_bytes(void);
size_t btb_b200_step_args_bytes(void);

#ifdef __cplusplus
}
#endif
#endif
