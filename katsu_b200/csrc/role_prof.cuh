// Per-role cycle accounting for tuning builds (-DKATSU_ROLE_PROF); compiled out otherwise.
// The including file defines KATSU_PROF_ARRAY (a device array name) and KATSU_PROF_READER
// (the extern "C" function that copies it to the host): [block][4 roles][4 phases] cycles.
#pragma once
#ifdef KATSU_ROLE_PROF
__device__ long long KATSU_PROF_ARRAY[256 * 16];
extern "C" int KATSU_PROF_READER(long long *out) {
    return (int)cudaMemcpyFromSymbol(out, KATSU_PROF_ARRAY, sizeof(long long) * 256 * 16);
}
#define PROF_DECL long long pt_[4] = {0, 0, 0, 0}, pc_ = clock64();
#define PROF_MARK(i) { const long long n_ = clock64(); pt_[i] += n_ - pc_; pc_ = n_; }
#define PROF_DUMP(slot) { for (int q_ = 0; q_ < 4; ++q_) KATSU_PROF_ARRAY[blockIdx.x * 16 + (slot) * 4 + q_] = pt_[q_]; }
#else
#define PROF_DECL
#define PROF_MARK(i) {}
#define PROF_DUMP(slot) {}
#endif
