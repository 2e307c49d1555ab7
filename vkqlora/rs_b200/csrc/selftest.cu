// Self-test entry points of the C ABI: they run pieces of the product kernels in isolation so that the
// parity tests can check them exhaustively (the NF4 code selection over every fp32 bit pattern) or drive
// a path that healthy runs never take (a bounded wait that gives up).  None has a counterpart in the
// reference.
#include "common.cuh"
#include "ptx.cuh"

namespace qlc {
namespace {

// One CTA, no TMA, no tensor memory: thread 0 waits on an mbarrier that nobody ever arrives on, with the
// same bounded wait the tensor-core kernels use but a short limit.  The wait gives up, raises the status
// word and the kernel returns normally.  Kernels queued behind it on the context see the raised status at
// their top and return without doing anything; qlc_ctx_synchronize reports and clears it.
__global__ void selftest_wait_timeout_kernel(DeviceStatus *status, long long limit_cycles, int site) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, status, site, limit_cycles);
        (void)ok;  // false: the limit ran out, the status word now says where
    }
    __syncthreads();
}

struct DevBuf {
    void *p = nullptr;
    ~DevBuf() {
        if (p) cudaFree(p);
    }
};

}  // namespace
}  // namespace qlc

using namespace qlc;

extern "C" {

int qlc_selftest_nf4_codes_of_targets(qlc_ctx *ctx, uint32_t first_bits, size_t count, uint8_t *out, size_t out_len) {
    if (!ctx) return fail(QLC_ERR_INVALID_CONFIG, "null context");
    if (out_len != (count + 1) / 2)
        return fail(QLC_ERR_SHAPE_MISMATCH, "out holds %zu bytes but ceil(count/2) = %zu", out_len, (count + 1) / 2);
    if ((uint64_t)first_bits + count > (1ull << 32)) return fail(QLC_ERR_INVALID_CONFIG, "bit patterns past 2^32");
    if (count == 0) return QLC_OK;
    if (!out) return fail(QLC_ERR_INVALID_CONFIG, "null output");
    QLC_CUDA(cudaSetDevice(ctx->device));
    DevBuf d;
    QLC_CUDA(cudaMalloc(&d.p, out_len));
    QLC_TRY(selftest_codes_of_targets(ctx, first_bits, count, static_cast<uint8_t *>(d.p)));
    QLC_CUDA(cudaMemcpyAsync(out, d.p, out_len, cudaMemcpyDeviceToHost, ctx->stream));
    return qlc_ctx_synchronize(ctx);
}

int qlc_selftest_nf4_fast_path(qlc_ctx *ctx, float absmax, uint32_t first_bits, uint64_t count, uint64_t *mismatches,
                               uint64_t *redone, uint32_t *first_mismatch_bits) {
    if (!ctx) return fail(QLC_ERR_INVALID_CONFIG, "null context");
    if ((uint64_t)first_bits + count > (1ull << 32)) return fail(QLC_ERR_INVALID_CONFIG, "bit patterns past 2^32");
    QLC_CUDA(cudaSetDevice(ctx->device));
    DevBuf d;
    QLC_CUDA(cudaMalloc(&d.p, 3 * sizeof(unsigned long long)));
    unsigned long long h[3] = {0ull, 0ull, ~0ull};
    QLC_CUDA(cudaMemcpyAsync(d.p, h, sizeof(h), cudaMemcpyHostToDevice, ctx->stream));
    QLC_TRY(selftest_fast_path(ctx, absmax, first_bits, count, static_cast<unsigned long long *>(d.p)));
    QLC_CUDA(cudaMemcpyAsync(h, d.p, sizeof(h), cudaMemcpyDeviceToHost, ctx->stream));
    QLC_TRY(qlc_ctx_synchronize(ctx));
    if (mismatches) *mismatches = h[0];
    if (redone) *redone = h[1];
    if (first_mismatch_bits) *first_mismatch_bits = h[0] ? (uint32_t)h[2] : 0u;
    return QLC_OK;
}

int qlc_selftest_wait_timeout(qlc_ctx *ctx, uint64_t limit_cycles) {
    if (!ctx) return fail(QLC_ERR_INVALID_CONFIG, "null context");
    // the limit is for tests of the failure path: at most ~50 ms of a B200's clock
    if (limit_cycles == 0 || limit_cycles > 100000000ull)
        return fail(QLC_ERR_INVALID_CONFIG, "limit_cycles must be in [1, 1e8]");
    QLC_CUDA(cudaSetDevice(ctx->device));
    selftest_wait_timeout_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_status, (long long)limit_cycles, 99);
    ctx->launches += 1;
    QLC_CUDA(cudaGetLastError());
    return QLC_OK;
}

}  // extern "C"
