// Launcher interface of the affine u4 matvec family (affine_matvec.cu).
#pragma once
#include "common.cuh"

namespace smelt {

enum AffineMode : int {
    kAffinePlain = 0,   // y = half(acc)                               affine_matvec
    kAffineAdd = 1,     // y = half(acc) + residual (fp16 add)         fused_affine_matvec_add
    kAffineGateUp = 2,  // y = half(silu(gate) * up), fp32 gate/up     fused_affine_gate_up_swiglu
    kAffineDual = 3,    // y = half(acc0), y2 = half(acc1)             fused_dual_affine_matvec
};

// One row range of a multi-tensor launch (plain mode only): e.g. Q | K | V sharing x.
struct AffineSeg {
    const uint8_t* w;
    const __half* s;
    const __half* b;
    __half* y;     // [batch, rows] of this segment
    int rows;      // a multiple of 16 for every segment but the last
};

struct AffineArgs {
    const uint8_t* w[2];   // packed nibbles [rows, cols/2]; [1] = up / second matrix
    const __half* s[2];    // scales [rows, cols/group]
    const __half* b[2];    // biases [rows, cols/group]
    const __half* x;       // activations [batch, cols]
    __half* y;             // [batch, rows]
    __half* y2;            // dual mode: second output
    const __half* residual;  // add mode: [batch, rows]; may alias y
    int rows, cols, batch;
    // Streaming kernel only.  norm_w != null: x is RMS-normalised while it is staged, with
    // the rounding points of rms_norm_1pw (half(x*rs) times half(1+w)).  nseg > 1: plain mode
    // over several tensors; rows is then the total row count.
    const __half* norm_w;
    float norm_eps;
    int nseg;
    AffineSeg seg[3];
    int ks, nsplit;        // filled by the launcher
    int sm_count;          // SMs of the device (0 = assume 148)
    // Tensor-memory QMM only: where CTAs that split a row tile's K leave their fp32 sums
    // (part_scratch_bytes bytes) and count their arrivals (one int per row tile, 4096 of them,
    // all zero between launches).  Launches that use them must not overlap on the device.
    float* part_scratch;
    size_t part_scratch_bytes;
    int* part_counters;
    uint32_t* err;         // device error word (may be null)
    DevDyn dyn;            // filled by the launcher
};

cudaError_t launch_affine(const Launch& l, int mode, const AffineArgs& args, int group);
cudaError_t launch_affine_stream(const Launch& l, int mode, const AffineArgs& args, int group, bool* handled);
// Tensor-memory QMM for batches of seventeen rows and more (affine_qmm.cu).
cudaError_t launch_affine_qmm(const Launch& l, int mode, const AffineArgs& args, int group, bool* handled);
// Wide-batch form (more than 64 rows of x): accumulates all of K in tensor memory (affine_qmm_wide.cu).
cudaError_t launch_affine_qmm_wide(const Launch& l, int mode, const AffineArgs& args, int group, bool* handled);
cudaError_t launch_affine_imma(const Launch& l, int mode, const AffineArgs& args, int group, bool* handled);

}  // namespace smelt
