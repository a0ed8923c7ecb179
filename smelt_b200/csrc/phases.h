// Multi-phase decode kernel: consecutive launches of a decode step that would each occupy the
// whole GPU for a few microseconds run as phases of one persistent cooperative kernel instead,
// separated by grid barriers.  A phase is exactly the device code of the stand-alone kernel
// (affine_imma.cuh, attention.cuh), so results do not change by a bit; what changes is that a
// CTA that finishes its share of phase p requests the first weight stages of phase p + 1 before
// it waits at the barrier, and that no launch, ramp and drain sits between the phases.
#pragma once
#include "affine_matvec.h"
#include "glue.h"

namespace smelt {

enum PhaseKind : int { kPhaseAffine = 0, kPhaseAttention = 1 };

struct Phase {
    int kind;    // PhaseKind
    int mode;    // affine: AffineMode
    union {
        AffineArgs affine;
        AttnDev attn;
    };
};

constexpr int kMaxPhases = 10;  // per launch: the argument block stays below the 4 KB kernel-parameter limit

struct PhaseProgram {
    int n;
    uint32_t* barrier;  // zero at launch
    uint32_t* err;      // device error word
    Phase ph[kMaxPhases];
};

struct PhaseRecorder {
    PhaseProgram prog;
    size_t smem = 0;        // largest dynamic shared memory any recorded phase needs
    uint32_t* barrier = nullptr;
    uint32_t* err = nullptr;
    int sm_count = 148;
    int launches = 0;       // multi-phase launches issued since the counters were last cleared
    int recorded = 0;       // phases recorded since then
};

// Appends a phase (flushing first when the program is full); smem = its dynamic shared memory.
cudaError_t record_affine_phase(const Launch& l, int mode, const AffineArgs& a, size_t smem);
cudaError_t record_attention_phase(const Launch& l, const AttnDev& p, size_t smem);
// Launches the recorded phases, if any, on the launch's stream.  Every real launch of a step
// calls it first, so stream order is the record order.
cudaError_t flush_phases(const Launch& l);

}  // namespace smelt
