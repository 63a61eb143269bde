/* CPU oracle for the KDA (Kimi delta attention) recurrent core.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain C++ restatement, in FP32, of the reference crate's CPU definitions
 * (crates/glm53f-kda/src/{bf16,synth,cpu,chunked}.rs).  It is the checker the parity tests, the smoke
 * test and the bench's CPU-baseline leg compare the CUDA kernels with; nothing that ships may call it.
 *
 * Pinning: the reference publishes no golden payloads for this path (its oracle/goldens manifests list
 * SHA-256 digests only), so the oracle is pinned by every known-answer value and invariant the reference's
 * own CPU tests assert (crates/glm53f-kda/tests/cpu_reference.rs, src/bf16.rs tests), reproduced in
 * tests/test_oracle_pins.py on the reference's own SplitMix64 streams.
 *
 * Layouts (elements, row-major):
 *   state, kernel layout   f32 [H][128 (v)][128 (k)]   (the C ABI's layout)
 *   state, literal layout  f32 [H][128 (k)][128 (v)]   (the transformers layout; kdao_transpose_state)
 *   conv window            f32 [3][C], C = 3*H*128, oldest row first
 *   conv weight            f32 [C][4], tap 3 multiplies the current row
 * All "bf16 tensors" are passed as f32 arrays holding bf16-exact values unless a name ends in _bits.
 */
#ifndef KDA_ORACLE_H
#define KDA_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { KDAO_FUSED = 0, KDAO_UNFUSED = 1, KDAO_F32 = 2 };

/* src/bf16.rs:6-23 */
uint16_t kdao_bf16_from_f32(float x);
float kdao_bf16_to_f32(uint16_t b);
float kdao_bf16_round(float x);
uint32_t kdao_bf16_ulp_distance(uint16_t a, uint16_t b);

/* src/synth.rs:10-45: SplitMix64, 24-bit uniforms.  `state` is the generator's 64-bit state. */
uint64_t kdao_rng_new(uint64_t seed);
uint64_t kdao_rng_next_u64(uint64_t* state);
void kdao_rng_fill(uint64_t* state, int64_t n, float lo, float hi, int round_bf16, float* out);

/* src/cpu.rs:203-254 */
float kdao_sigmoid(float x);
float kdao_silu(float x);
float kdao_warp_sum(const float* lanes32);
float kdao_dot128(const float* a, const float* b);
float kdao_log_decay(float a, float dt_bias, float a_log, float lower);
float kdao_decay(float a, float dt_bias, float decay_rate, float lower);
float kdao_beta(float b);

/* src/cpu.rs:304-376 (kernel order) and 557-568, 612-635 (literal order) */
void kdao_l2norm(const float* x, int has_scale, float scale, float* y);
void kdao_literal_l2norm(const float* x, float* y);
float kdao_q_scale(void);
void kdao_update(float* s, const float* k, const float* g, const float* v, float beta);
void kdao_read_out(const float* s, const float* q, float* y);
void kdao_gated_rmsnorm(const float* y, const float* norm_w, const float* gate, float eps, int mode, float* o);
void kdao_literal_gated_rmsnorm(const float* y, const float* norm_w, const float* gate, float eps, int mode, float* o);

/* src/cpu.rs:257-302: head h's q, k, v after conv + SiLU for row r of `rows`. */
void kdao_conv_qkv(int heads, const float* conv_w, const float* conv, const float* qkv, int r, int h, int mode,
                   float* q, float* k, float* v);

/* src/cpu.rs:380-471 (chain, chain_bf16_state) and 639-685 (literal::chain).  Outputs: out, y
 * [rows][H*128]; state_out [H][128][128] kernel layout; saves k,v,g [rows][H][128], beta [rows][H].
 * Any output pointer may be NULL. */
void kdao_chain(int heads, const float* conv_w, const float* a_log, const float* dt_bias, const float* norm_w,
                float eps, float lower, const float* conv, const float* state, int rows, const float* qkv,
                const float* a, const float* b, const float* gate, int mode, int bf16_state, int literal,
                float* out, float* y, float* state_out, float* k_save, float* v_save, float* g_save,
                float* b_save);

/* src/cpu.rs:475-508 */
void kdao_replay(int heads, const float* state, int rows_saved, const float* k_save, const float* v_save,
                 const float* g_save, const float* b_save, int keep, int bf16_state, float* state_out);

/* src/cpu.rs:512-527 */
void kdao_conv_shift(int heads, const float* conv, int rows, const float* qkv, int keep, float* out);

/* src/cpu.rs:531-547 */
void kdao_transpose_state(const float* s, int64_t n, float* t);

/* src/cpu.rs:573-610: one recurrent step on a literal-layout head state [128 (k)][128 (v)].
 * `normalize` != 0 runs lines 575-581 (L2-norm q and k, scale q); 0 takes q, k as given (the "core"
 * contract: q, k already normalised, scaled and rounded).  g is the log decay. */
void kdao_literal_step(float* s, const float* q, const float* k, const float* v, const float* g, float beta,
                       int normalize, float* y);

/* src/chunked.rs:67-198 (`head`): one head, literal-layout state, any chunk size. */
void kdao_chunked_head(int t, const float* q, const float* k, const float* v, const float* g, const float* beta,
                       float* state, int chunk, float* out);
/* src/chunked.rs:205-254 (`layer`): q,k,v [t][H][128] before the L2 norms, state [H][128 (k)][128 (v)]. */
void kdao_chunked_layer(int heads, int t, const float* q, const float* k, const float* v, const float* g,
                        const float* beta, float* state, int chunk, float* out);
/* src/chunked.rs:263-400 (`prefill_head`, the 16-row kernel's host model), kernel-layout head state. */
void kdao_prefill_head(int t, const float* qn, const float* kn, const float* v, const float* d, const float* beta,
                       float* s, float* y);
/* src/chunked.rs:405-467 (`prefill`): whole layer; outputs as kdao_chain without saves. */
void kdao_prefill(int heads, const float* conv_w, const float* a_log, const float* dt_bias, const float* norm_w,
                  float eps, float lower, const float* conv, const float* state, int rows, const float* qkv,
                  const float* a, const float* b, const float* gate, int mode, float* out, float* y,
                  float* state_out);

/* The "core" contract of the benchmark configurations: q, k, v bf16 bits [T][H][128] (q, k already
 * L2-normalised, q scaled), g f32 log decay [T][H][128], beta f32 [T][H]; state f32 in the KERNEL layout
 * [H][128 (v)][128 (k)], updated in place.  form 0 = the recurrence (kdao_literal_step with normalize = 0,
 * row by row), form 1 = kdao_chunked_head with `chunk`.  `y` receives the un-rounded read-out
 * [T][H][128] (may be NULL).  bf16_state != 0 rounds the state to bf16 after every row (form 0 only).
 * heads [h0, h1) are processed, on `threads` host threads. */
void kdao_core_forward(int heads, int h0, int h1, int64_t t, const uint16_t* q_bits, const uint16_t* k_bits,
                       const uint16_t* v_bits, const float* g, const float* beta, float* state, int form,
                       int chunk, int bf16_state, int threads, float* y);

/* The recurrent core in the KERNELS' operation order (src/cpu.rs:449-453 without the conv and the gates' own
 * arithmetic): for request b and each of its rows [cu_rows[b], cu_rows[b+1]): decay multipliers exp(g), optional
 * kernel-order L2 norms of q and k (src/cpu.rs:304-315), kdao_update, kdao_read_out rounded to bf16, then the
 * state rounded to bf16 when bf16_state.  State b lives at states + state_off[b], kernel layout, f32 values
 * (bf16-exact for bf16 states), updated in place.  y: bf16-rounded read-out [rows][H][128].  Optional saves as the
 * kernels write them.  Units (request, head) are spread over `threads` host threads. */
void kdao_core_step_batch(int heads, int batch, const int32_t* cu_rows, const uint16_t* q_bits, const uint16_t* k_bits,
                          const uint16_t* v_bits, const float* g, const float* beta, float* states,
                          const int64_t* state_off, int bf16_state, int l2norm, int threads, float* y, float* k_save,
                          float* v_save, float* g_save, float* b_save);

#ifdef __cplusplus
}
#endif
#endif
