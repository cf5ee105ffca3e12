// Context, error reporting and the small entry points of the C ABI.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <new>

#include "internal.h"

namespace iq {

int32_t fail(iq_ctx* ctx, int32_t code, const char* fmt, ...) {
    if (ctx != nullptr) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->last_error, sizeof(ctx->last_error), fmt, ap);
        va_end(ap);
    }
    return code;
}

int32_t check_cuda(iq_ctx* ctx, cudaError_t e, const char* what) {
    if (e == cudaSuccess) return kOk;
    return fail(ctx, kErrCuda, "%s: %s", what, cudaGetErrorString(e));
}

}  // namespace iq

using namespace iq;

extern "C" int32_t iq_abi_version(void) { return 1; }

extern "C" const char* iq_strerror(int32_t status) {
    switch (status) {
        case kOk: return "ok";
        case kErrInvalidArg: return "invalid argument";
        case kErrUnsupported: return "unsupported format or shape";
        case kErrCuda: return "CUDA error";
        case kErrWorkspace: return "workspace missing or too small";
        case kErrNoKernel: return "no kernel for this configuration";
        case kErrTimeout: return "device-side wait timed out";
        case kErrComm: return "communication error";
        case IQ_ERR_IO: return "file could not be opened, mapped or read";
        case IQ_ERR_FORMAT: return "not a safetensors file or inconsistent header";
        case IQ_ERR_MISSING: return "no such tensor";
        default: return "unknown status";
    }
}

extern "C" const char* iq_last_error(const iq_ctx* ctx) { return ctx ? ctx->last_error : "no context"; }

extern "C" int32_t iq_ctx_create(int32_t device, iq_ctx** out) {
    if (out == nullptr) return kErrInvalidArg;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) return kErrCuda;  // no CUDA device: there is no other path
    if (device < 0 || device >= count) return kErrInvalidArg;
    if (cudaSetDevice(device) != cudaSuccess) return kErrCuda;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return kErrCuda;
    if (prop.major != 10) return kErrUnsupported;  // the kernels are sm_100a only
    iq_ctx* ctx = new (std::nothrow) iq_ctx();
    if (ctx == nullptr) return kErrCuda;
    ctx->device = device;
    ctx->sms = prop.multiProcessorCount;
    ctx->smem_optin = (int)prop.sharedMemPerBlockOptin;
    cudaDriverEntryPointQueryResult qres;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
        ctx->encode_tiled = fn;
    int32_t st = kOk;
    if (cudaMalloc(&ctx->d_status, 256) != cudaSuccess || cudaMemset(ctx->d_status, 0, 256) != cudaSuccess) st = kErrCuda;
    // set-up time allocations of the GEMV's tail split: [slots][pieces][2 row sets][64] floats, [slots][blocks] counters
    const size_t tail_bytes = (size_t)iq::kQmvTailSlots * iq::kQmvTailPieces * 2 * 64 * sizeof(float);
    const size_t cnt_bytes = (size_t)iq::kQmvTailSlots * iq::kQmvTailBlocks * sizeof(uint32_t);
    if (st == kOk && (cudaMalloc(&ctx->qmv_tail_scratch, tail_bytes) != cudaSuccess ||
                      cudaMalloc(&ctx->qmv_tail_counters, cnt_bytes) != cudaSuccess ||
                      cudaMemset(ctx->qmv_tail_counters, 0, cnt_bytes) != cudaSuccess))
        st = kErrCuda;
    if (st == kOk) st = gqmv_init(ctx);
    if (st == kOk) st = qmm_init(ctx);
    if (st == kOk) st = moe_init(ctx);
    if (st == kOk) st = tern_init(ctx);
    if (st == kOk) st = w8a8_init(ctx);
    if (st != kOk) {
        if (ctx->d_status) cudaFree(ctx->d_status);
        if (ctx->qmv_tail_scratch) cudaFree(ctx->qmv_tail_scratch);
        if (ctx->qmv_tail_counters) cudaFree(ctx->qmv_tail_counters);
        delete ctx;
        return st;
    }
    *out = ctx;
    return kOk;
}

extern "C" void iq_ctx_destroy(iq_ctx* ctx) {
    if (ctx == nullptr) return;
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->qmv_tail_scratch) cudaFree(ctx->qmv_tail_scratch);
    if (ctx->qmv_tail_counters) cudaFree(ctx->qmv_tail_counters);
    delete[] ctx->qmv_maps;
    delete ctx;
}

extern "C" int32_t iq_ctx_set_wait_cycles(iq_ctx* ctx, uint64_t cycles) {
    if (ctx == nullptr) return kErrInvalidArg;
    if (cycles < 1000) return fail(ctx, kErrInvalidArg, "wait bound of %llu cycles (at least 1000)", (unsigned long long)cycles);
    ctx->wait_cycles = cycles;
    return kOk;
}

extern "C" int32_t iq_ctx_status(iq_ctx* ctx, int32_t* device_status) {
    if (ctx == nullptr || device_status == nullptr) return kErrInvalidArg;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return check_cuda(ctx, e, "cudaDeviceSynchronize");
    e = cudaMemcpy(device_status, ctx->d_status, 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return check_cuda(ctx, e, "cudaMemcpy(status)");
    if (*device_status != 0) cudaMemset(ctx->d_status, 0, 4);
    return kOk;
}
