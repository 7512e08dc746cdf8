// Parameters of the forward recurrence kernels (fwd.cu: inference and state-only runs; fwd_train.cu: the variant for a
// forward that keeps the per-chunk states and P_g tiles for a backward) and the launcher of the second one.
#pragma once
#include "host.cuh"
#include "seq.cuh"

namespace fq {

struct FwdParams {
  const float* g_cum;   // [rows, H] chunk-local cumsum of the log gate
  const float* beta;    // [rows, H]
  const float* h0;      // [n_h0, H, 128, 128] or nullptr
  float* ht;            // [n_out, H, 128, 128] or nullptr
  const int* ht_index;  // [n_seq] slot in ht per piece (negative: do not write) or nullptr (= piece index)
  const int* h0_index;  // [n_seq] slot in h0 per piece or nullptr (= piece index)
  const int* warmup;    // [n_entries, H] chunks to replay before the piece; bit 30 set = the replay starts at the
                        //            sequence start (use h0), else start from zero.  nullptr = {0 | bit 30}.
                        //            bit 29: start from h0_piece[piece] (no replay); bit 28: transition run (S = I and
                        //            the V tile ignored: the final state is the piece's transition matrix);
                        //            bit 27: nothing to do for this (entry, head)
  const int* piece_map; // [n_entries] piece of each grid entry, or nullptr (= entry); warmup and ht_index are per entry
  const float* h0_piece;  // [n_pieces, H, 128, 128] corrected start states (bit 29) or nullptr
  __nv_bfloat16* o;     // [rows, H, 128] or nullptr
  __nv_bfloat16* pg_out;  // [rows, H, 64] or nullptr: the P_g tiles, kept for the backward (only written together with o)
  __nv_bfloat16* h_out; // [total_chunks, H, 128(v), 128(k)] TRANSPOSED state before each chunk, or nullptr
                        // (written by TMA straight from the bf16 operand buffer)
  int H, Hg;
  float scale;
  SeqArgs sa;
  int* status_dev;
};

// gdr_fwd_train_kernel (fwd_train.cu): same arguments as gdr_fwd_kernel<false>; p.o and p.h_out must be given.
int launch_gdr_fwd_train(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& ma,
                         const CUtensorMap& mpg, const CUtensorMap& mh, const CUtensorMap& mo, const FwdParams& p,
                         unsigned ctas, cudaStream_t stream);

}  // namespace fq
