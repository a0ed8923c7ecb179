// The multi-phase decode kernel (see phases.h).
#include <cstring>

#include "affine_imma.cuh"
#include "attention.cuh"
#include "phases.h"

namespace smelt {

namespace {

constexpr int kThreads = 256;
constexpr uint32_t kBarrierSpinLimit = 1u << 21;  // about a second; then the error word gets bit 9 and the kernel carries on

// Grid barrier number `index` (1-based) of a launch whose counter started at zero.  The shape is
// that of a cooperative-groups grid sync: CTA barrier, one thread fences, arrives and polls,
// fences again, CTA barrier.
struct GridSync {
    uint32_t* counter;
    uint32_t* err;
    uint32_t target;  // 0: first phase of the launch, nothing to wait for
    __device__ __forceinline__ void operator()() const {
        if (target == 0) return;
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            atomicAdd(counter, 1u);
            uint32_t spins = 0;
            while (*reinterpret_cast<volatile uint32_t*>(counter) < target && ++spins < kBarrierSpinLimit) {}
            if (spins >= kBarrierSpinLimit && err) atomicOr(err, 0x200u);
            __threadfence();
        }
        __syncthreads();
    }
};

struct NoSync {
    __device__ __forceinline__ void operator()() const {}
};

__global__ void __launch_bounds__(kThreads, 1) decode_phases_kernel(const __grid_constant__ PhaseProgram prog) {
    extern __shared__ __align__(128) uint8_t smem[];
    for (int p = 0; p < prog.n; ++p) {
        const Phase& ph = prog.ph[p];
        const GridSync sync{prog.barrier, prog.err, p == 0 ? 0u : (uint32_t)p * gridDim.x};
        if (ph.kind == kPhaseAffine) {
            if (ph.mode == kAffinePlain) imma::affine_imma_body<kAffinePlain, 4, 8, 4, 1>(ph.affine, smem, sync);
            else if (ph.mode == kAffineAdd) imma::affine_imma_body<kAffineAdd, 4, 8, 4, 1>(ph.affine, smem, sync);
            else imma::affine_imma_body<kAffineGateUp, 3, 8, 4, 1>(ph.affine, smem, sync);
        } else {
            sync();
            const AttnDev& t = ph.attn;
            const int items = t.nsplits * t.a.n_kv * t.a.batch;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {
                const int split = item % t.nsplits, kvh = (item / t.nsplits) % t.a.n_kv, b = item / (t.nsplits * t.a.n_kv);
                attn::attn_decode_body<128, 1>(t, reinterpret_cast<float*>(smem), split, kvh, b, NoSync());
                __syncthreads();  // the next item reuses the shared memory
            }
        }
        __syncthreads();  // phases lay shared memory out differently: nobody starts the next one early
    }
}

}  // namespace

cudaError_t flush_phases(const Launch& l) {
    PhaseRecorder* r = l.phases;
    if (!r || r->prog.n == 0) return cudaSuccess;
    PhaseProgram prog = r->prog;
    prog.barrier = r->barrier;
    prog.err = r->err;
    const size_t smem = r->smem;
    r->prog.n = 0;
    r->smem = 0;
    cudaError_t e = cudaMemsetAsync(r->barrier, 0, sizeof(uint32_t), l.stream);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(decode_phases_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    prefer_max_shared(decode_phases_kernel);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(r->sm_count);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once, or the launch fails
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    r->launches += 1;
    return cudaLaunchKernelEx(&cfg, decode_phases_kernel, prog);
}

static cudaError_t make_room(const Launch& l) {
    return l.phases->prog.n == kMaxPhases ? flush_phases(l) : cudaSuccess;
}

cudaError_t record_affine_phase(const Launch& l, int mode, const AffineArgs& a, size_t smem) {
    cudaError_t e = make_room(l);
    if (e != cudaSuccess) return e;
    PhaseRecorder* r = l.phases;
    Phase& ph = r->prog.ph[r->prog.n++];
    r->recorded += 1;
    ph.kind = kPhaseAffine;
    ph.mode = mode;
    ph.affine = a;
    if (smem > r->smem) r->smem = smem;
    return cudaSuccess;
}

cudaError_t record_attention_phase(const Launch& l, const AttnDev& p, size_t smem) {
    cudaError_t e = make_room(l);
    if (e != cudaSuccess) return e;
    PhaseRecorder* r = l.phases;
    Phase& ph = r->prog.ph[r->prog.n++];
    r->recorded += 1;
    ph.kind = kPhaseAttention;
    ph.mode = 0;
    ph.attn = p;
    if (smem > r->smem) r->smem = smem;
    return cudaSuccess;
}

}  // namespace smelt
