// Shared helpers for the sm_100a kernels of the W4A4 linear path.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "../../include/quest_b200.h"

namespace qb {

// ---------------------------------------------------------------------------------------------
// Host-side helpers
// ---------------------------------------------------------------------------------------------
inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? QB200_OK : QB200_ERR_CUDA; }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Status of the launch just made.  The error (if any) is returned to the caller as a status code and
// cleared, so that it is not reported a second time by an unrelated later call.
// With QB200_DEBUG set in the environment the CUDA error text goes to stderr.
inline int launch_status() {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess && getenv("QB200_DEBUG") != nullptr) fprintf(stderr, "quest_b200: %s\n", cudaGetErrorString(e));
    return cuda_status(e);
}

// Programmatic dependent launches.  A kernel launched with `dependent` may be scheduled before the kernel that
// precedes it in the stream has completed (as soon as all of that kernel's blocks have executed
// griddepcontrol.launch_dependents or left); it must execute griddepcontrol.wait - which returns when the preceding grid
// has completed and its writes are visible - before its first access to global memory that the preceding kernel may
// write or still read.  Without the attribute both instructions do nothing.
__device__ __forceinline__ void wait_for_preceding_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void let_dependents_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename Kernel, typename... Args>
inline cudaError_t launch_kernel_dep(bool dependent, Kernel kernel, long long grid, int threads, size_t smem,
                                     cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// Set (per host thread) by the one-call layer entry points around their quantiser call: the tcgen05 quantiser kernel
// (which waits on the device) is then launched with a programmatic dependency.
extern thread_local bool qb_tl_dependent_quantiser;
// Which kernel the last hadamard_quantize_int4_cuda_bf16 call of this host thread launched (the one-call layer decides
// by it how to launch its GEMM).
constexpr int kQuantiserTc = 1, kQuantiserMma = 2;
extern thread_local int qb_tl_quantiser_kernel;

// Reads and clears the device status word of the row-kernel translation unit (see tcgen05.cuh).
int hq_tc_fetch_and_clear_device_status(int* out);

// Whether the tcgen05 quantiser can tile rows of K elements (block 128).
bool hq_tc_shape_ok(int K);

// ---------------------------------------------------------------------------------------------
// Device-side helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float bf16lo_to_f32(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// Two fp32 -> packed bf16x2 (round to nearest even); `lo` lands in bits [0,16).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ float bf16_to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

// Streaming 16-byte global load that does not allocate in L1 (data is read exactly once).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

// The Gaussian-MSE-optimal 4-bit clip constant and the derived step factor (2*c/15), and the eps,
// exactly as the reference evaluates them in fp32 (gemm-quest/quest/quantize_kernel.cu:81-86).
__device__ __forceinline__ float quest_scale_from_mean_square(float mean_sq) {
    const float factor = 2.513930578568423f * 2.f / 15.f;
    return sqrtf(mean_sq) * factor + 1e-8f;
}

}  // namespace qb
