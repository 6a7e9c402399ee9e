// A virtual thread block: the unit the small kernels are written for. A launch maps one CUDA block to it; a
// larger CTA could run several side by side, each with its own named barrier and slice of shared memory.
#pragma once

#include <cstdint>

struct VBlock {
    int x, y, z;          // block index in the operation's grid
    int tid;              // thread index inside the virtual block
    int nthreads;         // threads of the virtual block (a multiple of 32)
    int bar;              // named barrier id: 0 when the virtual block is the whole CTA
    unsigned char* smem;  // the block's private shared memory (16-byte aligned)

    __device__ __forceinline__ void sync() const {
        asm volatile("bar.sync %0, %1;\n" ::"r"(bar), "r"(nthreads) : "memory");
    }
};

// The virtual block of a standalone launch: the CUDA block itself.
__device__ __forceinline__ VBlock vblock_of_cta(unsigned char* dynamic_smem) {
    VBlock vb;
    vb.x = (int)blockIdx.x, vb.y = (int)blockIdx.y, vb.z = (int)blockIdx.z;
    vb.tid = (int)threadIdx.x;
    vb.nthreads = (int)blockDim.x;
    vb.bar = 0;
    vb.smem = dynamic_smem;
    return vb;
}
