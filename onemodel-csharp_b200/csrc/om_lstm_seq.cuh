// Whole-sequence LSTM kernels (om_lstm_seq.cu): parameter blocks and host entry points shared with om_recurrent.cu.
#pragma once
#include "om_common.cuh"

namespace om {

struct LstmSeqFwdDir {
  float* gates;          // [T, B, 4H]: in x W_ih^T, out the activated gates
  const float* w_hh;     // [4H, H]
  const float* bias;     // [4H] (b_ih + b_hh) or null
  const float* h0;       // [B, H] or null
  const float* c0;
  float* y;              // [T, B, H]
  float* c;
  float* tanh_c;
  unsigned* counter;     // barrier counts of this direction's row groups, zero at launch
  int reverse;
};
struct LstmSeqFwdParams {
  LstmSeqFwdDir d[2];
  int t, b, h;
  int passes, groups;    // a CTA covers passes x 16 batch rows; groups = row groups per direction
  int32_t* status;
};

struct LstmSeqBwdDir {
  const float* gates;    // [T, B, 4H] activated gates
  const float* tanh_c;   // [T, B, H]
  const float* c;
  const float* c0;       // [B, H] or null
  const float* gy;       // [T, B, H]
  const float* ghn;      // [B, H] or null
  const float* gcn;
  const float* w_hh;     // [4H, H]
  float* dG;             // [T, B, 4H] out
  float* dh0;            // [B, H] or null
  float* dc0;
  unsigned* counter;
  int reverse;
};
struct LstmSeqBwdParams {
  LstmSeqBwdDir d[2];
  int t, b, h;
  int passes, groups;
  int32_t* status;
};

// True when the context asks for the whole-sequence kernels (OM_SEQ_KERNELS), the shape fits them and all CTAs of
// `dirs` directions can be resident at once (the launch is cooperative).
bool lstm_seq_supported(om_ctx* ctx, int dirs, int t, int b, int h, bool backward);
// d[0..dirs-1] filled by the caller except `counter`.
int32_t lstm_seq_fwd(om_ctx* ctx, int dirs, int t, int b, int h, const LstmSeqFwdDir* d);
int32_t lstm_seq_bwd(om_ctx* ctx, int dirs, int t, int b, int h, const LstmSeqBwdDir* d);

}  // namespace om
