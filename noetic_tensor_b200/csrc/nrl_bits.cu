// The row forward and backward compiled for bit-packed vocabulary masks: bit v of a row is bit
// (v mod 32) of its 32-bit word v / 32. The kernel sources are the ones nrl_api.cu compiles; with
// NRL_MASK_BITS set their mask loads read one byte of bits per 8-element vector instead of eight
// mask bytes (common.cuh: ldg_mask8 and friends), and everything lands in namespace nrl_bits so
// that the two sets of kernels coexist in one library.
#define NRL_MASK_BITS 1
#define nrl nrl_bits
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "row_bwd.cuh"
#include "row_fwd_group.cuh"

using namespace nrl;

extern std::atomic<uint64_t> nrl_g_launches;

static inline int after_launch(int n = 1) {
    nrl_g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? NRL_OK : (int)e;
}

#define NRL_ROW_FWD_ENTRY nrl_row_fwd_bits
#define NRL_ROW_BWD_ENTRY nrl_row_bwd_bits
#include "row_api.inl"
