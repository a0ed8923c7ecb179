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

struct AffineArgs {
    const uint8_t* w[2];   // packed nibbles [rows, cols/2]; [1] = up / second matrix
    const __half* s[2];    // scales [rows, cols/group]
    const __half* b[2];    // biases [rows, cols/group]
    const __half* x;       // activations [batch, cols]
    __half* y;             // [batch, rows]
    __half* y2;            // dual mode: second output
    const __half* residual;  // add mode: [batch, rows]; may alias y
    int rows, cols, batch;
    int ks, nsplit;        // filled by the launcher
    int sm_count;          // SMs of the device (0 = assume 148)
    uint32_t* err;         // device error word (may be null)
    DevDyn dyn;            // filled by the launcher
};

cudaError_t launch_affine(const Launch& l, int mode, const AffineArgs& args, int group);
cudaError_t launch_affine_stream(const Launch& l, int mode, const AffineArgs& args, int group, bool* handled);

}  // namespace smelt
