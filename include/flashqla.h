/*
 * flashqla.h — C ABI of libflashqla_sm100.so: the chunked gated-delta-rule (GDN) kernels for
 * NVIDIA B200 (sm_100a).
 *
 * The reference project (FlashQLA) has no native interface: its kernels are JIT-generated from
 * Python and called through small torch wrappers.  Each entry point below replaces one of those
 * wrappers; the file:line given with it is the wrapper's location inside the FlashQLA project.
 *
 * Conventions (all entry points):
 *   - every pointer is a DEVICE pointer unless its name ends in `_host`;
 *   - tensors are dense row-major: q,k [B,T,Hg,128], v,o,do,dv [B,T,H,128], g,beta [B,T,H],
 *     A [B,T,H,64], states [n_seq,H,128,128] (K index before V index), h [total_chunks,H,128,128];
 *   - q/k/v/o/A/h are bfloat16, gates/beta fp32, states fp32;
 *   - variable-length batches: B == 1, `cu_seqlens` = int32 [n_seq+1] token offsets,
 *     `chunk_offsets` = int32 [n_seq+1] prefix sums of ceil(len/64); both NULL for dense batches
 *     (then n_seq == B and every sequence has T tokens);
 *   - the work is enqueued on `stream` (a cudaStream_t); nothing synchronises and nothing is allocated.
 *     The only state the library keeps between calls are per-device caches that are written once and never
 *     change afterwards (which kernels had their shared-memory limit raised, the SM count, the device address of
 *     the built-in scratch array of fq_gdr_bwd_chunk_gva_noalloc); they are filled under a mutex or with atomic,
 *     idempotent updates, so first calls from several host threads are safe.  A host thread's first call that
 *     builds tensor maps re-selects the current device through the runtime (cudaSetDevice) to bind the device's
 *     primary context to the thread: let each thread make its first call outside stream capture;
 *   - return value: 0 on success, negative FQ_ERR_* otherwise; fq_last_error() gives a message
 *     for the calling thread;
 *   - `status_dev` (may be NULL): int32 in device memory, must be 0 on entry; a kernel whose
 *     bounded wait expires stores a non-zero code there ((kernel id << 12) + wait site; the first expiry wins),
 *     stops waiting and runs to its end instead of hanging; the outputs of such a launch are meaningless.
 */
#ifndef FLASHQLA_H_
#define FLASHQLA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FQ_API __attribute__((visibility("default")))
#else
#define FQ_API
#endif

#define FQ_OK 0
#define FQ_ERR_INVALID (-1)
#define FQ_ERR_CUDA (-2)
#define FQ_ERR_UNSUPPORTED (-3)
#define FQ_ERR_WORKSPACE (-4)
#define FQ_ERR_TIMEOUT (-5)

/* Library version (major*100 + minor). */
FQ_API int fq_version(void);
/* Message of the last error raised on the calling thread. */
FQ_API const char* fq_last_error(void);

/*
 * Chunk-local (64-token) inclusive prefix sum of the log-gate, or suffix sum when reverse != 0.
 * Replaces chunk_local_cumsum, flash_qla/ops/utils/cumsum.py:131-165.
 * g, out: fp32 [B,T,H].  `out` may alias `g`.
 */
FQ_API int fq_chunk_cumsum(const float* g, float* out, int B, int T, int H, const int32_t* cu_seqlens,
                           const int32_t* chunk_offsets, int n_seq, int total_chunks, int reverse, void* stream);

/*
 * A = (I + strictly_lower(diag(beta) K K^T))^-1 per (chunk, V-head); gate-free, bf16 [B,T,H,64].
 * Rows of a partial tail chunk beyond the sequence end are not written.
 * Replaces kkt_solve, flash_qla/ops/gated_delta_rule/chunk/hopper/kkt_solve.py:305-345.
 */
FQ_API int fq_kkt_solve(const void* k, const float* beta, void* A, int B, int T, int H, int Hg,
                        const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq, int total_chunks,
                        void* stream);

/*
 * fq_kkt_solve that also emits the gated operand tiles of the recurrences (bf16 [B,T,H,64] each, NULL to skip):
 *   Ag[i][j] = A[i][j] * exp(g_i - g_j) * beta_j,   Pg[i][j] = scale * exp(g_i - g_j) * (q_i . k_j),   j <= i.
 * In the reference these products are formed inside the serial kernels
 * (flash_qla/ops/gated_delta_rule/chunk/hopper/fused_fwd.py:300-350); they are chunk-parallel, so here
 * they are produced by the chunk-parallel kernel.  g_cumsum: fp32 [B,T,H] from fq_chunk_cumsum.
 * a_is_input != 0: A is read instead of computed (the backward pass re-derives Ag / Pg from the A it was given).
 */
FQ_API int fq_kkt_solve_gated(const void* k, const void* q, const float* beta, const float* g_cumsum, void* A, void* Ag,
                              void* Pg, int a_is_input, int B, int T, int H, int Hg, const int32_t* cu_seqlens,
                              const int32_t* chunk_offsets, int n_seq, int total_chunks, float scale, void* stream);

/*
 * fq_chunk_cumsum + fq_kkt_solve_gated in one launch: `g` is the RAW log gate [B,T,H] fp32, its chunk-local
 * inclusive sum is formed per (chunk, V-head) inside the kernel (a warp scan), used for the gated tiles and written
 * to g_cumsum [B,T,H] fp32.  Saves the separate pass of flash_qla/ops/utils/cumsum.py:131-165 over g.
 * A may be NULL: the recurrence kernels do not read it, A is an input of the backward alone, so a forward that
 * will not be differentiated (prefill) need not write it.  Pg (and with it q) may be NULL: fq_gdr_fwd forms the
 * P_g tiles itself and can store them for the backward, which is cheaper than forming them here.
 */
FQ_API int fq_kkt_solve_fused(const void* k, const void* q, const float* beta, const float* g, float* g_cumsum, void* A,
                              void* Ag, void* Pg, int B, int T, int H, int Hg, const int32_t* cu_seqlens,
                              const int32_t* chunk_offsets, int n_seq, int total_chunks, float scale, void* stream);

/*
 * fq_kkt_solve_fused (without P_g) that also applies the activations of the caller's RAW gate and beta inputs while it
 * loads them, so that the elementwise passes a caller otherwise runs before the operator disappear
 * (flash_qla/ops/gated_delta_rule/chunk/__init__.py:30 takes an already activated g; the l2norm half of the same idea
 * is flash_qla/utils/math.py:7-21):
 *   gate_mode 0: g_raw is the log gate;  1: g = logsigmoid(g_raw);  2: g = -exp(A_log[h]) * softplus(g_raw + dt_bias[h])
 *             (A_log [H] fp32; dt_bias [H] fp32 or NULL);
 *   beta_mode 0: beta_raw is beta;  1: beta = sigmoid(beta_raw), also written to beta_out [B,T,H] fp32, which is what
 *             the recurrence and backward kernels then take as beta.
 * g_cumsum [B,T,H] receives the chunk-local sum of the ACTIVATED gate.  fq_gate_act_bwd is the backward of the
 * activations: dg / db (w.r.t. the activated values, as fq_gdr_bwd_chunk + the reverse fq_chunk_cumsum deliver them)
 * -> dg_raw / db_raw, and for gate mode 2 the per-head sums dA_log, ddt_bias ([H] fp32, ADDED to: zero them first;
 * either may be NULL).  db / beta_raw / db_raw may be NULL together.
 */
FQ_API int fq_kkt_solve_fused_act(const void* k, const float* beta_raw, const float* g_raw, const float* A_log,
                                  const float* dt_bias, int gate_mode, int beta_mode, float* g_cumsum, float* beta_out,
                                  void* A, void* Ag, int B, int T, int H, int Hg, const int32_t* cu_seqlens,
                                  const int32_t* chunk_offsets, int n_seq, int total_chunks, float scale, void* stream);
FQ_API int fq_gate_act_bwd(const float* dg, const float* db, const float* g_raw, const float* beta_raw, const float* A_log,
                           const float* dt_bias, int gate_mode, int beta_mode, float* dg_raw, float* db_raw, float* dA_log,
                           float* ddt_bias, long long rows, int H, void* stream);

/*
 * Fused forward recurrence: per (sequence, V-head) walks the chunks, carries the fp32 K x V state
 * and writes o = scale*exp(g) o (Q S) + P_g V_d per chunk.
 * Replaces fused_gdr_fwd, flash_qla/ops/gated_delta_rule/chunk/hopper/fused_fwd.py:535-658
 * (and, with o == NULL and h_out != NULL, the state-only fused_gdr_h of hopper/prepare_h.py:461-558).
 *   q,k [B,T,Hg,128] bf16; v [B,T,H,128] bf16; Ag [B,T,H,64] bf16 from fq_kkt_solve_gated / _fused;
 *   Pg [B,T,H,64] bf16 or NULL: an OUTPUT - the kernel forms P_g = scale * G o (Q K^T) of every chunk on its tensor
 *   core (the reference does the same inside its serial kernel, hopper/fused_fwd.py:300-350) and, if Pg is given
 *   together with o, stores the tiles for fq_gdr_bwd_dh / fq_gdr_bwd_chunk (rows past a sequence end are not written);
 *   g_cumsum, beta [B,T,H] fp32 (g_cumsum from fq_chunk_cumsum);
 *   h0   [n_seq,H,128,128] fp32 initial states, or NULL for zeros;
 *   ht   [*,H,128,128] fp32 final states, or NULL; sequence i writes slot ht_index[i]
 *        (negative = skip; ht_index == NULL means slot i);
 *   o    [B,T,H,128] bf16 or NULL;   h_out [total_chunks,H,128,128] bf16 (state BEFORE each chunk) or NULL.
 */
FQ_API int fq_gdr_fwd(const void* q, const void* k, const void* v, const void* Ag, void* Pg,
                      const float* g_cumsum, const float* beta, const float* h0, float* ht, const int32_t* ht_index,
                      void* o, void* h_out, int B, int T, int H, int Hg, const int32_t* cu_seqlens,
                      const int32_t* chunk_offsets, int n_seq, int total_chunks, float scale, int32_t* status_dev,
                      void* stream);

/*
 * fq_gdr_fwd with context-parallel pieces: `cu_seqlens` holds PIECE boundaries (pieces of one
 * sequence are contiguous and start on 64-token boundaries of their sequence).  Per piece:
 *   h0_index[i]  slot of h0 to start from when the replay reaches the sequence start (NULL = i);
 *   ht_index[i]  slot of ht to write, negative for non-terminal pieces (NULL = i);
 *   warmup[i*H+h] = w | (1<<30 if the replay starts at the sequence start): the CTA first replays the
 *                 w whole chunks before the piece (nothing stored) from h0 (bit 30) or from zero.  A piece may be
 *                 EMPTY (two equal boundaries): with w > 0 it is a state-only run over the w chunks in front of it and
 *                 its ht slot receives the state at that point of the sequence.
 * Replaces intra_card_cp_preprocess + correct_initial_states,
 * flash_qla/ops/gated_delta_rule/chunk/cp_context.py:106-163 and chunk/hopper/cp_fwd.py:256-309:
 * instead of computing per-piece end states in a separate pass and chaining them, every piece
 * warms its own state up inside the fused kernel.
 */
FQ_API int fq_gdr_fwd_cp(const void* q, const void* k, const void* v, const void* Ag, void* Pg,
                         const float* g_cumsum, const float* beta, const float* h0, float* ht, const int32_t* ht_index,
                         const int32_t* h0_index, const int32_t* warmup, void* o, void* h_out, int B, int T, int H,
                         int Hg, const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq, int total_chunks,
                         float scale, int32_t* status_dev, void* stream);

/*
 * fq_gdr_fwd_cp over a grid of `n_entries` entries instead of one per piece: entry e runs piece piece_map[e]
 * (NULL = e; mapped entries are state-only runs), `warmup` and `ht_index` are indexed by entry.  Further bits of
 * warmup[e*H+h]: bit 29 = start from h0_piece[piece] ([n_pieces,H,128,128] fp32) without replay; bit 28 =
 * transition run (state = identity, V ignored: the final state written to ht is the piece's K x K transition
 * matrix); bit 27 = nothing to do.  Together with fq_cp_transition_plan and fq_cp_chain this is the counterpart
 * of the (ht, mt) correction of flash_qla/ops/gated_delta_rule/chunk/hopper/cp_fwd.py:256-309, used for heads
 * whose gate decays too slowly for a replay.
 */
FQ_API int fq_gdr_fwd_cp_ex(const void* q, const void* k, const void* v, const void* Ag, void* Pg,
                            const float* g_cumsum, const float* beta, const float* h0, float* ht,
                            const int32_t* ht_index, const int32_t* h0_index, const int32_t* warmup,
                            const int32_t* piece_map, int n_entries, const float* h0_piece, void* o, void* h_out, int B,
                            int T, int H, int Hg, const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq,
                            int total_chunks, float scale, int32_t* status_dev, void* stream);

/*
 * Codes of the two forward passes for the (sequence, head) pairs flagged by fq_cp_warmup.
 *   warmup_in [n_pieces,H] from fq_cp_warmup (reverse == 0); piece_seq / chunks_before / chunks_after [n_pieces];
 *   flags [n_seq,H] as left by the scan(s): a backward pass runs both directions into the same flags.
 *   warmup_out [n_pieces,H]: codes of the final pass (bit 29 for every piece but the first of a flagged pair).
 *   pass1_codes [2*n_pieces,H]: entry r = end state of piece r from zero (from h0 for a first piece), entry
 *   n_pieces + r = transition matrix of piece r; bit 27 where not needed.
 */
FQ_API int fq_cp_transition_plan(const int32_t* warmup_in, const int32_t* piece_seq, const int32_t* chunks_before,
                                 const int32_t* chunks_after, const int32_t* flags, int32_t* warmup_out,
                                 int32_t* pass1_codes, int n_pieces, int H, void* stream);

/*
 * fq_cp_warmup (one or both directions) and fq_cp_transition_plan(_reverse) in ONE launch: a CTA per (sequence, head)
 * scans the replay length of every piece of that pair, derives the flag and writes the codes.
 *   piece_start / piece_end [n_pieces]: first token of / after the piece; chunks_before / chunks_after [n_pieces];
 *   last_chunk_len [n_pieces]: tokens in the last chunk of the piece's sequence; seq_piece_offsets [n_seq+1].
 *   flags [n_seq,H], codes [n_pieces,H], pass1_codes [2*n_pieces,H] as documented at fq_cp_transition_plan;
 *   codes_rev / pass1_rev [n_pieces,H] (both or neither): the tables of the state-gradient recurrence, a pair being
 *   flagged when the replay of either direction exceeds w_cap chunks.
 */
FQ_API int fq_cp_plan(const float* g_cumsum, const int32_t* piece_start, const int32_t* piece_end,
                      const int32_t* chunks_before, const int32_t* chunks_after, const int32_t* last_chunk_len,
                      const int32_t* seq_piece_offsets, int32_t* flags, int32_t* codes, int32_t* pass1_codes,
                      int32_t* codes_rev, int32_t* pass1_rev, int n_pieces, int n_seq, int H, float threshold, int w_cap,
                      void* stream);

/*
 * h0_piece[r+1] = T_r h0_piece[r] + B_r along the pieces of every flagged (sequence, head), in fp32.
 *   bt [2*n_pieces,H,128,128]: B_r in slot r, T_r in slot n_pieces + r (the ht of the pass-1 run);
 *   seq_piece_offsets [n_seq+1]: first piece of every sequence.
 */
FQ_API int fq_cp_chain(const float* bt, float* h0_piece, const int32_t* flags, const int32_t* seq_piece_offsets,
                       int n_pieces, int n_seq, int H, void* stream);

/*
 * The chain kernel behind fq_cp_chain / fq_cp_chain_reverse with its two further modes; `add` and `tmat` are given
 * separately ([n_pieces,H,128,128] fp32 each, indexed by piece), `out` has one slot per piece:
 *   reverse == 0: out[r+1] = T_r out[r] + add[r] for the pieces r of every flagged (sequence, head); the first step
 *                 takes add alone (the first piece's end state already contains the sequence's initial state);
 *   reverse != 0: out[r-1] = T_r^T out[r] + add[r] from the last piece down; the first step takes add alone;
 *   init    (optional, [H,128,128] fp32): the chain starts from this state (gradient) instead, and every step, the
 *                 first included, applies its transition matrix;
 *   compose != 0 (forward only, add unused): the product of the transition matrices alone, out[first+1] = T_first,
 *                 out[r+1] = T_r out[r] - the K x K transition of a whole run of pieces.
 * seq_piece_offsets may name one piece more than exists (offsets [0, P+1] over P pieces): the forward chain then also
 * delivers the state after the last piece in out[P].  This is how one GPU's share of a sequence is summarised as
 * (end state from zero, transition matrix) for the exchange between GPUs; the reference chains the same pair between
 * the pieces of one card (flash_qla/ops/gated_delta_rule/chunk/hopper/cp_fwd.py:144-165).
 */
FQ_API int fq_cp_chain_ex(const float* add, const float* tmat, float* out, const int32_t* flags,
                          const int32_t* seq_piece_offsets, const float* init, int n_seq, int H, int reverse, int compose,
                          void* stream);

/*
 * Gate scan for context-parallel pieces (counterpart of get_warmup_chunks,
 * flash_qla/ops/gated_delta_rule/chunk/hopper/cp_fwd.py:69-101).  For every (piece, head) returns in
 * warmup[piece*H+h] the number of whole chunks adjacent to the piece that must be replayed so that
 * older history has decayed below exp(threshold); bit 30 is set when the replay reaches the end of
 * the sequence (then it is exact and starts from the sequence's boundary state).
 *   reverse == 0 (forward state): piece_edge = first token of the piece, piece_aux = chunks that
 *                precede the piece in its sequence; piece_chunks_after unused.
 *   reverse != 0 (state gradient): piece_edge = first token after the piece, piece_chunks_after =
 *                chunks that follow the piece in its sequence, piece_aux = token count of the
 *                sequence's last chunk.
 *   w_cap > 0 bounds the walk: a replay longer than w_cap chunks is reported as w_cap + 1 (no bit 30) without
 *                looking further; 0 = walk to the end.
 *   flags [n_seq,H] (optional, zeroed by the caller; needs piece_seq [n_pieces] = sequence of each piece and a cap):
 *                set to 1 for every (sequence, head) with a piece whose replay exceeds w_cap chunks.
 */
FQ_API int fq_cp_warmup(const float* g_cumsum, const int32_t* piece_edge, const int32_t* piece_aux,
                        const int32_t* piece_chunks_after, int32_t* warmup, int n_pieces, int H, float threshold,
                        int reverse, int w_cap, const int32_t* piece_seq, int32_t* flags, void* stream);

/*
 * Backward, serial part: reverse recurrence of the state gradient per (sequence, V-head).
 * Together with fq_gdr_bwd_chunk it replaces fused_gdr_bwd,
 * flash_qla/ops/gated_delta_rule/chunk/hopper/fused_bwd.py:900-985.
 *   Ag, Pg [B,T,H,64] bf16 from fq_kkt_solve_gated;
 *   dout [B,T,H,128] bf16 (gradient of o); dht [n_seq,H,128,128] fp32 or NULL (gradient of the final state);
 *   dh0  [n_seq,H,128,128] fp32 or NULL (gradient of the initial state);
 *   dh_out [total_chunks,H,128(v),128(k)] bf16: gradient w.r.t. the state AFTER each chunk, stored transposed
 *   (scratch for fq_gdr_bwd_chunk).
 */
FQ_API int fq_gdr_bwd_dh(const void* q, const void* k, const void* Ag, const void* Pg, const void* dout,
                         const float* g_cumsum, const float* beta, const float* dht, float* dh0, void* dh_out, int B,
                         int T, int H, int Hg, const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq,
                         int total_chunks, float scale, int32_t* status_dev, void* stream);

/*
 * fq_gdr_bwd_dh over context-parallel pieces (`cu_seqlens` = piece boundaries, see fq_gdr_fwd_cp):
 *   dht_index[i] slot of dht used when the replay reaches the end of the sequence; dh0_index[i] slot of dh0
 *   to write (negative for pieces that do not start their sequence); seq_end[i] first token after the
 *   piece's sequence; warmup[i*H+h] chunks to replay AFTER the piece (from fq_cp_warmup, reverse != 0).
 * The reference has no context parallelism in its backward.
 */
FQ_API int fq_gdr_bwd_dh_cp(const void* q, const void* k, const void* Ag, const void* Pg, const void* dout,
                            const float* g_cumsum, const float* beta, const float* dht, float* dh0, void* dh_out,
                            const int32_t* dht_index, const int32_t* dh0_index, const int32_t* seq_end,
                            const int32_t* warmup, int B, int T, int H, int Hg, const int32_t* cu_seqlens,
                            const int32_t* chunk_offsets, int n_seq, int total_chunks, float scale,
                            int32_t* status_dev, void* stream);

/*
 * fq_gdr_bwd_dh_cp with corrected start gradients: bit 29 of warmup[i*H+h] = start piece i from
 * dht_piece[i] ([n_pieces,H,128,128] fp32: the gradient at the piece's end) with no replay; bit 27 = nothing to do.
 * fq_cp_transition_plan_reverse makes the codes of the two launches for the pairs flagged by
 * fq_cp_transition_plan: the gradient pass (every piece but the first of its sequence from zero, the last one from
 * dht; its dh0 slots give C_r) and the final pass; fq_cp_chain_reverse forms e_{r-1} = T_r^T e_r + C_r from the last
 * piece down, with the transition matrices T_r of the forward state pass (tmat = bt + n_pieces*H*128*128).
 */
FQ_API int fq_gdr_bwd_dh_cp_ex(const void* q, const void* k, const void* Ag, const void* Pg, const void* dout,
                               const float* g_cumsum, const float* beta, const float* dht, float* dh0, void* dh_out,
                               const int32_t* dht_index, const int32_t* dh0_index, const int32_t* seq_end,
                               const int32_t* warmup, const float* dht_piece, int B, int T, int H, int Hg,
                               const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq, int total_chunks,
                               float scale, int32_t* status_dev, void* stream);
FQ_API int fq_cp_transition_plan_reverse(const int32_t* warmup_in, const int32_t* piece_seq,
                                         const int32_t* chunks_before, const int32_t* chunks_after, const int32_t* flags,
                                         int32_t* warmup_out, int32_t* pass1_codes, int n_pieces, int H, void* stream);
FQ_API int fq_cp_chain_reverse(const float* c, const float* tmat, float* dht_piece, const int32_t* flags,
                               const int32_t* seq_piece_offsets, int n_pieces, int n_seq, int H, void* stream);

/*
 * Backward, chunk-parallel part: dv (bf16 [B,T,H,128]), dq, dk (per V-head, bf16 [B,T,H,128]), dg w.r.t. the
 * gate cumsum and dbeta (fp32 [B,T,H]) from h (state before each chunk, from fq_gdr_fwd with h_out; stored
 * transposed [.., 128(v), 128(k)]) and dh (from fq_gdr_bwd_dh, same layout).
 * Second half of the replacement of hopper/fused_bwd.py:900-985.
 */
FQ_API int fq_gdr_bwd_chunk(const void* q, const void* k, const void* v, const void* A, const void* Ag,
                            const void* Pg, const void* dout, const void* h, const void* dh, const float* g_cumsum,
                            const float* beta, void* dq, void* dk, void* dv, float* dg, float* db, int B, int T, int H,
                            int Hg, const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq, int total_chunks,
                            float scale, int32_t* status_dev, void* stream);

/*
 * fq_gdr_bwd_chunk with the sum over the V-heads of every QK head done inside the kernel: dq, dk are [B,T,Hg,128]
 * (the reference sums them after its kernel with group_reduce_vector,
 * flash_qla/ops/gated_delta_rule/chunk/__init__.py:107-110; tests/ref_gdr.py:694-698).
 * A CTA takes the V-heads of a (chunk, QK head) pair one after the other, stores the first head's tile and ADDS the
 * others' (TMA reduce; tail chunks row by row), in that fixed order: for two V-heads per QK head the result is
 * bit-identical to fq_gdr_bwd_chunk + fq_group_reduce_pair, and the [B,T,H,128] per-head copies are never written.
 */
FQ_API int fq_gdr_bwd_chunk_grouped(const void* q, const void* k, const void* v, const void* A, const void* Ag,
                                    const void* Pg, const void* dout, const void* h, const void* dh,
                                    const float* g_cumsum, const float* beta, void* dq, void* dk, void* dv, float* dg,
                                    float* db, int B, int T, int H, int Hg, const int32_t* cu_seqlens,
                                    const int32_t* chunk_offsets, int n_seq, int total_chunks, float scale,
                                    int32_t* status_dev, void* stream);

/*
 * fp32 correction of dg at the two ends of every sequence, applied between fq_gdr_bwd_chunk and the reverse
 * fq_chunk_cumsum.  dg of a chunk's last token contains gamma_last * sum(dS o S0) over the 128 x 128 state;
 * fq_gdr_bwd_chunk forms it from the bf16 copies h / dh.  For a sequence's first chunk S0 is the caller's fp32 h0, for
 * its last chunk dS is the caller's fp32 dht: this adds the products with the rounding residuals (h0 - bf16(h0),
 * dht - bf16(dht)) to dg_cum in place, which makes the term exact for one-chunk sequences.  h0 / dht may be NULL.
 * The reference keeps dS in fp32 registers inside its one serial kernel
 * (flash_qla/ops/gated_delta_rule/chunk/hopper/fused_bwd.py:335-357); this is what the split into two kernels owes.
 *   h, dh [total_chunks,H,128(v),128(k)] bf16; h0, dht [n_seq,H,128,128] fp32; g_cumsum, dg_cum [B,T,H] fp32.
 */
FQ_API int fq_dg_boundary_fix(const float* h0, const float* dht, const void* h, const void* dh, const float* g_cumsum,
                              float* dg_cum, int B, int T, int H, const int32_t* cu_seqlens,
                              const int32_t* chunk_offsets, int n_seq, int total_chunks, void* stream);

/*
 * out[r, hg, :] = sum of in[r, hg*G .. hg*G+G-1, :] (G = H / Hg), bf16 in/out, fp32 accumulation.
 * Replaces group_reduce_vector, flash_qla/ops/utils/group_reduce.py:60-79.
 */
FQ_API int fq_group_reduce(const void* in, void* out, long long rows, int H, int Hg, void* stream);
/* The same for two tensors of one shape in ONE launch (dq and dk of the backward, which the reference sums with
 * two calls, flash_qla/ops/gated_delta_rule/chunk/__init__.py:104-107). */
FQ_API int fq_group_reduce_pair(const void* in_a, void* out_a, const void* in_b, void* out_b, long long rows, int H,
                                int Hg, void* stream);

/*
 * y = x * rsqrt(sum(x^2 over the last dim) + eps) for rows of 128 bf16 values, and its backward
 * dx = r dy - x r^3 (x . dy).  Replaces l2norm, flash_qla/utils/math.py:7-21 (a torch.compile'd elementwise
 * function there, applied to q and k when use_qk_l2norm_in_kernel is set, chunk/__init__.py:221-223).
 */
FQ_API int fq_l2norm_fwd(const void* x, void* y, long long rows, float eps, void* stream);
FQ_API int fq_l2norm_bwd(const void* x, const void* dy, void* dx, long long rows, float eps, void* stream);

/*
 * Token-by-token recurrence (decode / short continuations): consumes the final state written by fq_gdr_fwd
 * (flash_qla/ops/gated_delta_rule/chunk/hopper/fused_fwd.py:214-221 writes it, :173-179 reads it back as
 * initial_state) and advances it by T tokens per sequence.  The reference has no such operator (prefill and
 * training only); the arithmetic is the token-level form of the same recurrence:
 *   S <- e^g S;  v' = beta (v - S^T k);  S <- S + k v'^T;  o = scale S^T q.
 *   q, k [N,T,Hg,128] bf16; v, o [N,T,H,128] bf16; g (log gate, NOT cumulated), beta [N,T,H] fp32;
 *   state_in [N,H,128,128] fp32 or NULL (zero); state_out [N,H,128,128] fp32 or NULL; may alias state_in.
 */
FQ_API int fq_gdr_recurrent(const void* q, const void* k, const void* v, const float* g, const float* beta,
                            const float* state_in, float* state_out, void* o, int N, int T, int H, int Hg, float scale,
                            void* stream);

/*
 * Allocation-free variant of fq_gdr_bwd_chunk + fq_group_reduce for grouped heads; it has no
 * counterpart in the reference.  Same inputs as fq_gdr_bwd_chunk, but dq and dk are the final
 * [B,T,Hg,128] gradients: the per-V-head partial results that the regular path keeps in two
 * caller-allocated [B,T,H,128] buffers are held in a 32 MiB array inside the library instead.
 * It exists for callers that must not allocate device memory where the backward runs (a step whose
 * buffers were all planned in advance and whose allocator is frozen, or a host that would
 * otherwise pay a device-synchronising cudaMalloc per call).
 *   - limit: B*T*H <= 65536; larger problems return FQ_ERR_WORKSPACE with a message;
 *   - cost: the 32 MiB array is part of the library image, so every GPU on which the library is loaded holds it
 *     from load until the process exits, whether or not this entry point is ever called;
 *   - the first call on each device resolves the array's device address and configures the kernel;
 *     make that first call outside any stream capture (and see the note on a thread's first call above);
 *   - all calls share the one array and it keeps the previous call's contents: nothing in it has to
 *     be cleared (every row is rewritten before it is read), but two calls that overlap on the GPU
 *     (different streams, or different host threads) race on it; serialise them;
 *   - it allocates nothing: no cudaMalloc, no cudaFree of a buffer, no allocating library routine.
 */
FQ_API int fq_gdr_bwd_chunk_gva_noalloc(const void* q, const void* k, const void* v, const void* A, const void* Ag,
                                        const void* Pg, const void* dout, const void* h, const void* dh,
                                        const float* g_cumsum, const float* beta, void* dq, void* dk, void* dv,
                                        float* dg, float* db, int B, int T, int H, int Hg, const int32_t* cu_seqlens,
                                        const int32_t* chunk_offsets, int n_seq, int total_chunks, float scale,
                                        int32_t* status_dev, void* stream);

/*
 * Self-test of the tensor-core plumbing (TMA 128B-swizzled tiles -> UMMA -> TMEM -> registers).
 * a, b: bf16 [128,128] row-major; d: fp32 [128,128].  `mode` selects the operand forms, see
 * csrc/selftest.cu.  No counterpart in the reference; used by the GPU tests only.
 */
FQ_API int fq_selftest_umma(const void* a, const void* b, float* d, int mode, int32_t* status_dev, void* stream);

/*
 * Self-test of the bounded waits: launches one small CTA in which one warp waits, for at most `limit_cycles`
 * (1 .. 1e8), on an mbarrier that nothing completes.  Expected: *status_dev (0 on entry) becomes
 * (14 << 12) + 5 = 0xE005, the other warps' waits end as soon as the abort flag is up, the CTA releases its
 * tensor memory and writes 1 to *done_dev; the context stays usable.  No counterpart in the reference (its
 * TileLang kernels wait without a bound); used by the GPU tests only.
 */
FQ_API int fq_selftest_wait_expiry(int32_t* status_dev, int32_t* done_dev, long long limit_cycles, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASHQLA_H_ */
