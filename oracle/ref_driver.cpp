/*
 * TEST INFRASTRUCTURE ONLY — never linked into, imported by, or called from the product library.
 *
 * Launcher for the reference kernels compiled as host C++ (see ref_shim.h).
 *
 * ref_launch(fn, nthreads, nargs, args) calls one reference kernel body on `nthreads` host
 * threads.  Thread t runs the body with blockIdx.x = t, gridDim.x = nthreads, blockDim.x = 1,
 * threadIdx.x = 0; because every reference kernel is a grid-stride loop
 * (`for (i = blockIdx.x*blockDim.x + threadIdx.x; i < n; i += blockDim.x*gridDim.x)`), the
 * union over t visits each index once, which is what the reference's GPU launch
 * `<<<ceil(n/128),128>>>` (reference cuda/src/kernels/binary.rs:78-97) does too.
 *
 * Every parameter of every reference entry point except the alpha/beta pair of
 * add_alpha_beta_inplace_* is an integer-class value of at most 8 bytes (size_t, int64_t,
 * bool, pointers), so the arguments are passed as an array of uint64_t and forwarded through
 * a ten-integer-argument function pointer; on the 64-bit SysV and AAPCS64 calling conventions
 * surplus integer arguments are ignored by the callee.
 */
#include <cstdint>
#include <cstring>
#include <omp.h>

struct ref_dim3 {
    unsigned int x, y, z;
};
thread_local ref_dim3 blockIdx = {0, 0, 0};
thread_local ref_dim3 threadIdx = {0, 0, 0};
thread_local ref_dim3 blockDim = {1, 1, 1};
thread_local ref_dim3 gridDim = {1, 1, 1};

typedef void (*fn10_t)(uint64_t, uint64_t, uint64_t, uint64_t, uint64_t, uint64_t, uint64_t, uint64_t, uint64_t,
                       uint64_t);

extern "C" int ref_max_threads() { return omp_get_max_threads(); }

extern "C" int ref_launch(void* fn, int nthreads, int nargs, const uint64_t* args) {
    if (!fn || nargs < 0 || nargs > 10) return 1;
    uint64_t a[10];
    std::memset(a, 0, sizeof(a));
    for (int i = 0; i < nargs; i++) a[i] = args[i];
    if (nthreads < 1) nthreads = 1;
    fn10_t f = reinterpret_cast<fn10_t>(fn);
#pragma omp parallel num_threads(nthreads)
    {
        const int t = omp_get_thread_num();
        const int nt = omp_get_num_threads();
        blockIdx = {static_cast<unsigned>(t), 0, 0};
        threadIdx = {0, 0, 0};
        blockDim = {1, 1, 1};
        gridDim = {static_cast<unsigned>(nt), 1, 1};
        f(a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], a[8], a[9]);
    }
    return 0;
}
