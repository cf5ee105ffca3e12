/*
 * ingot_qmm.h — C ABI of libingot_qmm.so: ingot's quantized-matmul hot path (MLX affine 4/8-bit g64 and MXFP4
 * quantized linear layers; decode GEMV, prefill GEMM, MoE grouped form) as hand-written CUDA for NVIDIA B200 (sm_100a).
 *
 * The reference engine (Swift + Metal) has no FFI; this header is what a Swift module map (include/module.modulemap,
 * module CIngotQMM) would import so that the bodies of the reference's four launcher entry points can call CUDA where
 * they dispatched Metal kernels. Each declaration cites the reference interface it replaces (paths inside the
 * reference project).
 *
 * Conventions, kept from the reference:
 *   - weights stay in the MLX layout byte for byte (Sources/Ingot/Loader/Quant.swift:4-12): `w` uint32
 *     [experts, n, k*bits/32] with value j of a row in bits [bits*j, bits*j+bits); `scales`/`biases` bf16
 *     [experts, n, k/group] (affine, w = scale*q + bias) or `scales` uint8 e8m0 [experts, n, k/32] and no biases (mxfp4);
 *   - every pointer is a device pointer owned by the caller; nothing is allocated, freed or synchronised in a call that
 *     takes a stream: work is enqueued on `stream` (a cudaStream_t passed as void*) and the call returns;
 *   - scratch memory is the caller's (one exception: the decode GEMV's tail scratch, see iq_qmv): ask for the size once (…_workspace_bytes), allocate it at layer construction
 *     (the reference allocates its scratch at construction too, Layers/MoE.swift:220-241), pass it to every call;
 *   - every function returns 0 or a negative iq_status; iq_last_error(ctx) gives the message. Shapes the reference's
 *     launchers reject with a precondition (rows > 16 in qmv, M % 64 != 0 in qmm, …) come back as IQ_ERR_INVALID_ARG;
 *   - a context serves one device; calls on one context from several threads must use different streams and may not
 *     share workspaces.
 * There is no CPU path: every entry point either enqueues CUDA kernels or fails.
 */
#ifndef INGOT_QMM_H
#define INGOT_QMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct iq_ctx iq_ctx;
typedef struct iq_moe iq_moe;

typedef enum iq_status {
    IQ_OK = 0,
    IQ_ERR_INVALID_ARG = -1, /* a shape / pointer / flag the operator does not accept */
    IQ_ERR_UNSUPPORTED = -2, /* a format or combination with no kernel (the reference's "load error") */
    IQ_ERR_CUDA = -3,        /* a CUDA runtime call failed; see iq_last_error */
    IQ_ERR_WORKSPACE = -4,   /* workspace missing or too small */
    IQ_ERR_NO_KERNEL = -5,
    IQ_ERR_TIMEOUT = -6, /* a bounded device-side wait gave up (status word written by the kernel) */
    IQ_ERR_COMM = -7,
    IQ_ERR_IO = -8,      /* loader: a file could not be opened, mapped or read */
    IQ_ERR_FORMAT = -9,  /* loader: not a safetensors file / inconsistent header */
    IQ_ERR_MISSING = -10 /* loader: no such tensor */
} iq_status;

typedef enum iq_dtype { IQ_F32 = 0, IQ_F16 = 1, IQ_BF16 = 2 } iq_dtype;
typedef enum iq_mode { IQ_MODE_AFFINE = 0, IQ_MODE_MXFP4 = 1 } iq_mode;
/* FFN activations, numbered as the reference's lab_glu (qmm.metal:9-31): SiLU gate, GELU (tanh form) gate, gpt-oss's
 * clamped swiglu_oai, and relu^2 of the up projection alone (the gate tensor is then the up tensor, MoE.swift:130-133). */
typedef enum iq_act { IQ_ACT_SILU = 0, IQ_ACT_GELU = 1, IQ_ACT_SWIGLU_OAI = 2, IQ_ACT_RELU2 = 3 } iq_act;
typedef enum iq_router_kind { IQ_ROUTER_BF16 = 0, IQ_ROUTER_Q8 = 1 } iq_router_kind;
/* How the router scores experts (RouterSpec, Loader/ModelSpecParts.swift:64; kernels verify.metal:181-260 and
 * ab_moe_route.metal:20-53): softmax over the chosen logits, or a sigmoid per expert with an optional bias that only
 * steers the selection and weights p / (sum of the chosen p + eps). */
typedef enum iq_router_score { IQ_SCORE_SOFTMAX = 0, IQ_SCORE_SIGMOID = 1 } iq_router_score;
/* Shared expert: none, with a sigmoid gate per token, or with weight 1 (LAB_MOE_SHARED 0 / 1 / 2, verify.metal:165). */
typedef enum iq_shared_kind { IQ_SHARED_NONE = 0, IQ_SHARED_GATED = 1, IQ_SHARED_UNGATED = 2 } iq_shared_kind;

enum {
    IQ_FLAG_ACCUMULATE = 1, /* y += result (VQMV.encode accumulate:, encodeQmmF32 accumulate:) */
    IQ_FLAG_NO_BARRIER = 2  /* iq_linear_colsplit: leave the flag barriers out (the host orders the ranks itself) */
};

/* A quantized matrix on the device. Replaces DenseQ (Sources/Ingot/Layers/Linear.swift:17-33) and
 * DeviceQuantizedLinear (Sources/Ingot/Loader/Quant.swift:205-231): three buffers plus N, K, bits, group size.
 * `experts` > 1: stacked expert tensors, expert e at word offset e*n*(k*bits/32) and scale offset e*n*(k/group). */
typedef struct iq_qlinear {
    const void* w;
    const void* scales;
    const void* biases; /* NULL for mxfp4 */
    int32_t n;          /* output features (rows of W) */
    int32_t k;          /* input features */
    int32_t bits;       /* 4 or 8; 6 for the decode GEMV (k a multiple of 2048) and the embedding; 2 = the rotated
                           ternary format: group 128, `scales` fp16, biases unused (w = (q - 1) * scale), activations
                           rotated by iq_had_rows first (Shaders/xc_tern.metal) */
    int32_t group;      /* 64 (affine; 32 also for the 4-bit decode GEMV and the embedding), 128 (ternary) or 32 (mxfp4) */
    int32_t mode;       /* iq_mode */
    int32_t experts;    /* leading dimension, 1 for a plain layer */
} iq_qlinear;

/* ---- context -------------------------------------------------------------------------------------------------------
 * Replaces MetalContext (Sources/Ingot/GPU.swift:6-29: one device, one queue, the pipeline cache). Creating a context
 * selects the device, checks that it is sm_100 and configures the kernels' shared-memory limits. */
int32_t iq_ctx_create(int32_t device, iq_ctx** out);
void iq_ctx_destroy(iq_ctx* ctx);
const char* iq_strerror(int32_t status);
const char* iq_last_error(const iq_ctx* ctx);
/* Synchronises the device and returns the status word that kernels with bounded waits write when a wait gives up
 * (0 = none did; the word is cleared when read). The reference surfaces GPU errors at waitUntilCompleted
 * (Sources/Ingot/GPU.swift:164-167); this is the equivalent place. Not for the enqueue path. */
int32_t iq_ctx_status(iq_ctx* ctx, int32_t* device_status);
/* Bound, in SM clock cycles, of the waits on another GPU (the flag barriers of the expert-parallel exchange and of the
 * column-split linear). The default, 4e9 cycles, is about two seconds; a host that watches its peers itself (a
 * heartbeat) can shorten it so that a rank whose peer has gone comes back within milliseconds with IQ_ERR_TIMEOUT in
 * iq_ctx_status. The reference has no counterpart (one GPU, no peer to wait for). Applies to calls enqueued afterwards. */
int32_t iq_ctx_set_wait_cycles(iq_ctx* ctx, uint64_t cycles);
/* ABI version of this header (bumped on incompatible changes). */
int32_t iq_abi_version(void);

/* ---- decode GEMV ---------------------------------------------------------------------------------------------------
 * Y[rows, n] (+)= X[rows, k] * W^T, rows <= 16. Replaces VQMV.encode(enc, x:, xOffset:, xFloat:, m, y:, yOffset:, rows:,
 * ldx:, ldy:, accumulate:, nPrefix:) (Sources/Ingot/Layers/Linear.swift:287-444) and the kernels behind it
 * (Shaders/verify_nax.metal:105-209, Shaders/verify.metal:89-155).
 * x: [rows, ldx] of x_dtype (the reference takes half or float; bf16 is added because the checkpoints' activations
 * are bf16); y: [rows, ldy] of y_dtype (the reference writes float). n_prefix > 0 computes only the first n_prefix
 * output features (a multiple of 16). Requires n % 16 == 0, k % 64 == 0, ldx % 8 == 0, 16-byte aligned x.
 * The bits of activation row i do not depend on `rows` or on the other rows (for a given n_prefix: a call over a prefix
 * of the output features may sum an output feature's K slices in another order than a call over all of them).
 * Scratch: matrices whose 16-row blocks do not divide over the GPU's CTAs sum a few left-over blocks through a small
 * scratch area that the context owns (the one exception to "scratch is the caller's": a few hundred KB allocated at
 * iq_ctx_create). Each stream that makes such calls holds one of 16 slots of it for the life of the context; a 17th
 * stream is refused with IQ_ERR_INVALID_ARG. A CUDA graph keeps the slot of the stream it was captured on: two graphs
 * captured on the same stream must not be replayed at the same time. */
int32_t iq_qmv(iq_ctx* ctx, void* stream, const void* x, int32_t x_dtype, int64_t ldx, const iq_qlinear* m, void* y,
               int32_t y_dtype, int64_t ldy, int32_t rows, uint32_t flags, int32_t n_prefix);

/* ---- prefill GEMM --------------------------------------------------------------------------------------------------
 * Y[rows, n] (+)= X[rows, k] * W^T on the tcgen05 tensor cores (weights dequantised to fp16 in shared memory, fp32
 * accumulation in tensor memory). Replaces DenseQ.encodeQmmF32(ctx, enc, x:, xOffset:, y:, rows:, accumulate:, halfOut:)
 * (Sources/Ingot/Layers/Linear.swift:688-713) and qmm_t_nax3* (Shaders/qmm_nax_v3.metal:107-256).
 * Requires rows % 64 == 0 and n % 64 == 0 like the reference (Linear.swift:695), k % 64 == 0.
 * x of dtype bf16/f32 is converted to fp16 into the workspace first; fp16 x is used in place. */
int32_t iq_qmm_workspace_bytes(iq_ctx* ctx, const iq_qlinear* m, int32_t rows, int32_t x_dtype, size_t* bytes);
int32_t iq_qmm(iq_ctx* ctx, void* stream, const void* x, int32_t x_dtype, int64_t ldx, const iq_qlinear* m, void* y,
               int32_t y_dtype, int64_t ldy, int32_t rows, uint32_t flags, void* workspace, size_t workspace_bytes);

/* Prefill GEMM for callers that must not allocate device memory. No counterpart in the reference (its scratch is
 * ordinary Metal buffers made at construction). Meant for hosts where cudaMalloc is off limits at the call site: a
 * plugin inside an engine whose pool owns all device memory, a path that runs after the pool is sealed, a sandbox or
 * real-time loop with a "no allocation" rule. Same operation and results as iq_qmm, but the fp16 copy of bf16/fp32
 * activations goes to an 8 MiB array built into the library (held by every GPU that loads it until the process
 * exits) instead of a caller workspace. Limits and rules:
 *   - rows * k <= 4,194,304 (8 MiB of fp16); larger calls return IQ_ERR_WORKSPACE and should use iq_qmm;
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress) with that device current;
 *     make that first call outside any stream capture;
 *   - the call itself allocates and frees nothing;
 *   - all calls on a GPU share the one array: calls whose kernels may overlap on the GPU (different streams) race on
 *     it — keep them on one stream or order them. Nothing in it has to be cleared between calls. */
int32_t iq_qmm_noalloc(iq_ctx* ctx, void* stream, const void* x, int32_t x_dtype, int64_t ldx, const iq_qlinear* m,
                       void* y, int32_t y_dtype, int64_t ldy, int32_t rows, uint32_t flags);

/* Rotated W8A8 prefill GEMM (lossy; an option of the serving path, not the default). Replaces DenseQ.encodeQmmI8(ctx, enc,
 * x:, y:, rows:, scratch:, accumulate:, halfOut:) (Sources/Ingot/Layers/Dense.swift:99-172) and w4_i8rot /
 * quant_rows_rot_i8g / qmm_i8 (Shaders/xa_dense_i8.metal): per call the 4-bit weights and the activations are rotated
 * along K (unnormalised Hadamard of 256 inputs per block when k / 32 is a multiple of 32, else of 32), quantised to int8
 * per row, and Y = (Xq Wq^T) sx sw / n runs on the int8 tensor cores. The workspace (the reference's DenseI8Scratch)
 * holds the int8 weights [n, k], the int8 activations [rows, k] and both scale vectors. 4-bit affine weights
 * (group 64 or 32), rows and n multiples of 64, k a multiple of 128. Bound of the reference's int8-serve case
 * (Tests/IngotTests/KernelCaseTests.swift:623-661): relative RMS error 2e-3 against the CPU emulation of the same
 * arithmetic, 5e-2 against the exact product.
 * A ternary matrix (bits 2, group 128) takes DenseQ.encodeQmmI8T instead (Dense.swift:174-212; quant_rows_i8 and
 * tern_i8row, Shaders/xc_tern.metal:189-237): x is the input already rotated by iq_had_rows and goes to int8 per row
 * with no further rotation, a weight row goes to int8 with one scale, s_row = max_g |s_g| / 127, as t * rint(s_g / s_row),
 * and Y = (Xq Wq^T) sx sw. Bounds of the reference's bonsai-int8 case (Tests/IngotTests/KernelCaseFlashNextI8.swift
 * :155-213): relative RMS error 2e-3 against the emulation, 3e-2 against the exact product. */
int32_t iq_qmm_w8a8_workspace_bytes(iq_ctx* ctx, const iq_qlinear* m, int32_t rows, size_t* bytes);
int32_t iq_qmm_w8a8(iq_ctx* ctx, void* stream, const void* x, int32_t x_dtype, int64_t ldx, const iq_qlinear* m, void* y,
                    int32_t y_dtype, int64_t ldy, int32_t rows, uint32_t flags, void* workspace, size_t workspace_bytes);

/* ---- dense gated FFN ------------------------------------------------------------------------------------------------
 * out[rows, d] (+)= down( act(gate x) * up x ) with gate|up concatenated by rows as one [2*d_ff, d] matrix (gate rows
 * first). Replaces DenseMLP.encode / encodePrefill (Sources/Ingot/Layers/Dense.swift:56-96) and dswiglu*
 * (Shaders/yy_model.metal:187-227). rows <= 16 takes the GEMV path, larger multiples of 64 the GEMM path. */
int32_t iq_dense_ffn_workspace_bytes(iq_ctx* ctx, const iq_qlinear* gate_up, const iq_qlinear* down, int32_t rows,
                                     int32_t x_dtype, size_t* bytes);
int32_t iq_dense_ffn(iq_ctx* ctx, void* stream, const void* x, int32_t x_dtype, int64_t ldx, const iq_qlinear* gate_up,
                     const iq_qlinear* down, int32_t act, float act_limit, void* out, int32_t out_dtype, int64_t ldo,
                     int32_t rows, uint32_t flags, void* workspace, size_t workspace_bytes);

/* ---- MoE layer -----------------------------------------------------------------------------------------------------
 * Replaces MoELayer (Sources/Ingot/Layers/MoE.swift:54-429) and PrefillMoE (Sources/Ingot/Layers/MoEPrefill.swift:29-278):
 * router -> top-k -> group by expert -> gate+up+activation -> down -> weighted combine. The description is the
 * reference's load-time state: RouterSpec (Loader/ModelSpecParts.swift:64), the stacked expert tensors, the optional
 * gpt-oss expert biases (MoEPrefill.swift:9-22). Accepted shapes are the reference's (MoE.swift:186-219,
 * MoEPrefill.swift:129-142): experts % 32 == 0, experts <= 512, top_k <= 16, d_ff % 64 == 0, d_model % 64 == 0,
 * d_model >= 128, experts affine 4-bit g64 or mxfp4, router bf16 or 8-bit g64; anything else is IQ_ERR_UNSUPPORTED. */
typedef struct iq_moe_desc {
    int32_t experts;        /* E: experts of the model (router width) */
    int32_t top_k;
    int32_t d_model;
    int32_t d_ff;
    int32_t act;            /* iq_act */
    float act_limit;        /* swiglu_oai clamp (the config's swiglu_limit, 7) */
    int32_t router_kind;    /* iq_router_kind */
    float routed_scale;     /* multiplies the renormalised weights (routed_scaling_factor); 1 when absent */
    const void* router_w;   /* bf16 [E, d_model], or uint32 8-bit codes [E, d_model/4] */
    const void* router_scales;      /* 8-bit router only */
    const void* router_biases;      /* 8-bit router only */
    const float* router_logit_bias; /* fp32 [E] added to the logits (gpt-oss mlp.router.bias) or NULL */
    const float* per_expert_scale;  /* fp32 [E] (Gemma 4 router.per_expert_scale) or NULL */
    iq_qlinear gate;        /* [local experts, d_ff, d_model] */
    iq_qlinear up;          /* [local experts, d_ff, d_model] */
    iq_qlinear down;        /* [local experts, d_model, d_ff] */
    const float* gate_bias; /* fp32 [local experts, d_ff] or NULL */
    const float* up_bias;   /* fp32 [local experts, d_ff] or NULL */
    const float* down_bias; /* fp32 [local experts, d_model] or NULL */
    int32_t expert_lo;      /* first expert held here (expert parallel); 0 on one GPU */
    int32_t expert_count;   /* experts held here; == experts on one GPU. The reference's analogue is the
                               expert->slot table `smap` (MoE.swift:104) */
    int32_t router_score;   /* iq_router_score */
    float route_eps;        /* sigmoid scoring: added to the sum of the chosen scores before the division */
    const float* router_select_bias; /* sigmoid scoring: fp32 [E] added to the scores for the selection only
                                        (e_score_correction_bias) or NULL */
    /* Shared expert (MoE.swift:140-154): one more FFN that every token goes through, 4-bit affine g64, its own width
     * (shared_gate_proj.n); out += w_s * down_s(act(gate_s x, up_s x)) with w_s = sigmoid(x . shared_gate) or 1. */
    int32_t shared;                  /* iq_shared_kind */
    iq_qlinear shared_gate_proj;     /* [1, d_ff_s, d_model] (relu^2: pass the up tensor) */
    iq_qlinear shared_up;            /* [1, d_ff_s, d_model] */
    iq_qlinear shared_down;          /* [1, d_model, d_ff_s] */
    iq_qlinear shared_gate;          /* IQ_SHARED_GATED: 8-bit affine g64 [1, 1, d_model], the gate's logit weights */
} iq_moe_desc;

/* Pieces of a forward call, for timing and for callers that run an exchange between them. The names are the
 * reference's (MoELayer.Piece MoE.swift:328; PrefillMoE.Piece MoEPrefill.swift:55). */
enum {
    IQ_PIECE_ROUTER = 1,  /* logits = x * router^T */
    IQ_PIECE_ROUTE = 2,   /* top-k indices and weights */
    IQ_PIECE_GROUP = 4,   /* token -> expert permutation, tile list */
    IQ_PIECE_GATEUP = 8,  /* h = act(gate x, up x) per expert */
    IQ_PIECE_DOWN = 16,   /* yd = down h per expert */
    IQ_PIECE_COMBINE = 32, /* out (+)= sum_k w * yd */
    IQ_PIECE_ALL = 63
};

/* Device views into the workspace after a forward call (valid until the next call with the same workspace). */
typedef struct iq_moe_views {
    float* logits;      /* [T, ld], ld = experts rounded up to 64 (MoELayer.routerLD, MoE.swift:296) */
    int32_t ld;
    uint32_t* inds;     /* [T, top_k] expert ids, descending score, ties to the lower id */
    float* wts;         /* [T, top_k] */
    uint32_t* offsets;  /* [E + 1] first sorted position of each expert */
    uint32_t* row_map;  /* [T*top_k] sorted position -> pair id (pair = token*top_k + rank) */
    uint32_t* pos;      /* [T*top_k] pair id -> sorted position */
    void* h;            /* fp16 [T*top_k, d_ff] activations at sorted positions */
    void* yd;           /* [T*top_k, d_model] expert outputs at sorted positions: fp16 for affine experts, fp32 for
                           MXFP4 ones, whose outputs can pass half's range (the reference's choice, MoEPrefill.swift:159) */
    int32_t yd_dtype;   /* IQ_F16 or IQ_F32 */
} iq_moe_views;

int32_t iq_moe_create(iq_ctx* ctx, const iq_moe_desc* desc, iq_moe** out);
void iq_moe_destroy(iq_moe* layer);
/* Workspace for up to `max_tokens` tokens per call. */
int32_t iq_moe_workspace_bytes(const iq_moe* layer, int32_t max_tokens, size_t* bytes);
/* out[T, ldo] (+)= MoE(x[T, ldx]). Replaces MoELayer.encode(enc, x:, out:, rows:, accumulate:, only:)
 * (MoE.swift:346-428) for any T and PrefillMoE.encode / encodeAll (MoEPrefill.swift:173-278). `pieces` is a mask of
 * IQ_PIECE_*; a partial mask reuses what earlier pieces left in the workspace. */
int32_t iq_moe_forward(iq_moe* layer, void* stream, const void* x, int32_t x_dtype, int64_t ldx, void* out,
                       int32_t out_dtype, int64_t ldo, int32_t tokens, uint32_t flags, uint32_t pieces, void* workspace,
                       size_t workspace_bytes);
/* Routing only, on logits the caller supplies ([T, ld] fp32): writes inds [T, top_k] and wts [T, top_k].
 * Replaces the route kernels as the reference's router cases drive them (Tests/IngotTests/KernelCaseRouter.swift:110-126). */
int32_t iq_moe_route(iq_moe* layer, void* stream, const float* logits, int32_t ld, int32_t tokens, uint32_t* inds,
                     float* wts);
/* Routing set by the caller for the next forward calls (PrefillMoE.externalRouting, MoEPrefill.swift:80-86): device
 * arrays inds [T, top_k], wts [T, top_k]; pass NULLs to go back to the layer's own router. */
int32_t iq_moe_set_external_routing(iq_moe* layer, const uint32_t* inds, const float* wts);
int32_t iq_moe_get_views(const iq_moe* layer, void* workspace, int32_t tokens, iq_moe_views* out);

/* ---- expert parallelism --------------------------------------------------------------------------------------------
 * The reference runs on one GPU and has no counterpart for these (its nearest notion is the expert -> slot table
 * `smap`, Layers/MoE.swift:104). With experts sharded in contiguous ranges over the ranks of one box, a layer is:
 *   sender:   iq_moe_forward(ROUTER|ROUTE|GROUP) on its tokens, iq_moe_pack_rows -> rows in expert order, which is
 *             one contiguous segment per destination rank; all-to-all of the rows (the host's collective);
 *   owner:    iq_moe_experts on the rows it received (source-major, expert order inside a source) -> yd rows;
 *             all-to-all back;
 *   sender:   iq_moe_combine_rows on the returned rows, in its own expert order.
 * Routing is computed by every rank for its own tokens with the full router, so indices do not depend on the number
 * of ranks. */
/* rows_f16[pos[pair], :] = fp16(x[pair / top_k, :]) for the routing that GROUP left in `workspace`. */
int32_t iq_moe_pack_rows(iq_moe* layer, void* stream, const void* x, int32_t x_dtype, int64_t ldx, int32_t tokens,
                         void* workspace, size_t workspace_bytes, void* rows_f16);
int32_t iq_moe_experts_workspace_bytes(const iq_moe* layer, int32_t max_rows, int32_t sources, size_t* bytes);
/* Gate/up/activation/down of the layer's own experts on received rows. rows_f16: fp16 [max_rows, d_model] of which
 * the first sum(counts) rows are live; total_rows is the caller's (expected or exact) row count and only picks the
 * kernels, every bound comes from max_rows and the device-side counts;
 * counts: device uint32 [sources, experts], counts[s*experts + e] = rows source s sent for expert e (rows are ordered
 * by source, then expert: packed one source after the other when region_rows == 0, or source s starting at row
 * s*region_rows); yd: fp16 or fp32, same row positions. yd_rows (device array of max_rows addresses, or null): when
 * given, the output of row r goes to yd_rows[r] (d_model elements of yd_dtype, 16-byte aligned, any memory this GPU can
 * store to, a peer's included; 0 = row unused) by a copy kernel that follows the experts, and yd is scratch. */
int32_t iq_moe_experts(iq_moe* layer, void* stream, const void* rows_f16, int32_t total_rows, int32_t max_rows,
                       const uint32_t* counts, int32_t sources, int32_t region_rows, void* yd, int32_t yd_dtype,
                       void* const* yd_rows, void* workspace, size_t workspace_bytes);
/* The same for rows left where they arrived: row i of the expert-major order (sum(counts) rows, experts ascending) is
 * row row_index[i] of rows_f16 (device array of max_rows entries, e.g. from iq_ep_index); the kernels fetch the rows
 * through the index, so nothing is gathered first. counts: device uint32 [experts] (one source). */
int32_t iq_moe_experts_indexed(iq_moe* layer, void* stream, const void* rows_f16, const uint32_t* row_index, int32_t total_rows,
                               int32_t max_rows, const uint32_t* counts, void* yd, int32_t yd_dtype, void* const* yd_rows,
                               void* workspace, size_t workspace_bytes);
/* out[t, :] (+)= sum_k wts[t, k] * yd_rows[pos[t*top_k + k], :] with the routing in `workspace`. */
int32_t iq_moe_combine_rows(iq_moe* layer, void* stream, const void* yd_rows, int32_t yd_dtype, int32_t tokens, void* out,
                            int32_t out_dtype, int64_t ldo, uint32_t flags, void* workspace, size_t workspace_bytes);

/* Device-side exchange: the same layer with no host involvement, so that a multi-layer step can live in one CUDA
 * graph. The host allocates, once, four buffers per rank in memory every peer can address (cudaIpc / cuMem / torch
 * symmetric memory) and passes the peers' addresses: recv (fp16 [world * region_rows, d_model]: region s holds the rows
 * source rank s sends, in local-expert order, so region_rows >= the largest tokens*top_k of any rank), back (expert
 * outputs returning, [tokens*top_k, d_model] of yd_dtype), flags (uint32 [world], zeroed) and counts (uint32
 * [world, experts]). Per layer, on every rank, in stream order:
 *   iq_moe_forward(ROUTER|ROUTE|GROUP); iq_ep_pack_push; iq_ep_barrier(then_plan = 1);
 *   iq_moe_experts(recv, counts = own counts matrix, region_rows); iq_ep_return_push; iq_ep_barrier(0);
 *   (or, faster: iq_ep_index, then iq_moe_experts_indexed(recv, row_index, merged counts, yd_rows = table), and no
 *   iq_ep_return_push: the experts fetch the rows through the index and their outputs go from yd straight into the
 *   sources' return buffers through the table; iq_ep_compact gathers the rows first instead)
 *   iq_moe_combine_rows(back).
 * Rows move with plain 16-byte peer stores (no TMA, no multicast). Every rank must run the same sequence; the barrier's
 * wait is bounded (IQ_ERR_TIMEOUT in iq_ctx_status when a peer never arrives). At most 8 ranks. */
typedef struct iq_ep iq_ep;
int32_t iq_ep_create(iq_ctx* ctx, int32_t rank, int32_t world, int32_t experts, int32_t region_rows,
                     void* const* peer_recv, void* const* peer_back, void* const* peer_flags, void* const* peer_counts,
                     iq_ep** out);
void iq_ep_destroy(iq_ep* ep);
/* Writes this rank's per-expert row counts (offsets[e+1] - offsets[e]) into row `rank` of every peer's counts matrix
 * (iq_ep_pack_push does the same; this entry point serves hosts that move the rows themselves). */
int32_t iq_ep_share_counts(iq_ep* ep, void* stream, const uint32_t* offsets);
/* All ranks meet; with then_plan != 0 the kernel then derives the return-path plan from the completed counts matrix. */
int32_t iq_ep_barrier(iq_ep* ep, void* stream, int32_t then_plan);
/* The plan alone (after a barrier that followed the sharing of the counts). */
int32_t iq_ep_plan(iq_ep* ep, void* stream);
/* fp16 rows of this rank's tokens, in expert order, stored straight into region `rank` of the owners' receive buffers,
 * together with this rank's counts; needs nothing from the peers. tokens*top_k <= region_rows. */
int32_t iq_ep_pack_push(iq_ep* ep, void* stream, const void* x, int32_t x_dtype, int64_t ldx, int32_t tokens,
                        int32_t top_k, int32_t d_model, const uint32_t* inds, const uint32_t* pos, const uint32_t* offsets);
/* Expert outputs of the received rows ([world * region_rows, d_model], the layout of recv) stored back into each
 * source's return buffer at the source's sorted positions. */
int32_t iq_ep_return_push(iq_ep* ep, void* stream, const void* yd, int32_t yd_dtype, int32_t d_model);
/* The same mapping as a table for iq_moe_experts' yd_rows (device array of world * region_rows addresses). */
int32_t iq_ep_return_rows(iq_ep* ep, void* stream, int32_t yd_dtype, int32_t d_model, void** table);
/* Received rows gathered out of their regions into expert-major order (rows_out, fp16 [world * region_rows, d_model]):
 * all sources' rows of one expert end up next to each other, so the grouped GEMM dequantises each weight tile once per
 * expert rather than once per (source, expert). table gets the return address of every compacted row (for yd_rows);
 * *merged_counts is a device array [experts] of this rank's per-expert row totals: pass it to iq_moe_experts as counts
 * with sources = 1, region_rows = 0. After iq_ep_barrier(then_plan = 1). */
int32_t iq_ep_compact(iq_ep* ep, void* stream, const void* recv_rows, int32_t d_model, int32_t yd_dtype, void* rows_out,
                      void** table, const uint32_t** merged_counts);
/* The same order without moving the rows: row_index[i] = the receive-buffer row at position i of the expert-major order
 * (device array of world * region_rows entries), table and merged_counts as in iq_ep_compact; for
 * iq_moe_experts_indexed(recv, row_index, ...). Faster: the rows are read once, by the experts' kernels. */
int32_t iq_ep_index(iq_ep* ep, void* stream, int32_t d_model, int32_t yd_dtype, uint32_t* row_index, void** table,
                    const uint32_t** merged_counts);
/* The dispatch with every token row sent once per destination rank, however many of its experts live there (top-8
 * routing over 2 / 4 / 8 ranks: 4 / 2.2 / 1.5 pairs per token and rank reached, so that many times fewer bytes cross
 * NVLink). The receive buffer then holds fp16 rows [world * tok_rows, d_model] (row s * tok_rows + t = token t of
 * source s; tok_rows >= the largest token count of any rank, the same value on every rank) followed by the token of
 * every received pair; iq_ep_index_tokens turns that into the row index iq_moe_experts_indexed takes. Sequence as
 * above with iq_ep_pack_push_tokens for iq_ep_pack_push and iq_ep_index_tokens for iq_ep_index. */
int32_t iq_ep_pack_push_tokens(iq_ep* ep, void* stream, const void* x, int32_t x_dtype, int64_t ldx, int32_t tokens,
                               int32_t top_k, int32_t d_model, const uint32_t* inds, const uint32_t* pos,
                               const uint32_t* offsets, int32_t tok_rows);
int32_t iq_ep_index_tokens(iq_ep* ep, void* stream, int32_t d_model, int32_t yd_dtype, int32_t tok_rows, uint32_t* row_index,
                           void** table, const uint32_t** merged_counts);

/* ---- column-split dense linear ---------------------------------------------------------------------------------------
 * One dense quantized linear over the GPUs of one box: rank r holds output features [r*n/G, (r+1)*n/G) (rows of w /
 * scales / biases: one contiguous byte range of each tensor), x is replicated, every rank ends up with the whole y.
 * The reference runs on one GPU and has no counterpart; a shard is what its row concatenation and nPrefix calls address
 * (Layers/Linear.swift:107-183, 350-366). The host allocates, once, on every rank, y ([max_rows, n] of y_dtype, row
 * pitch n) and flags (uint32 [world], zeroed) in memory every peer can address and passes all ranks' addresses.
 * iq_linear_colsplit, on every rank, in stream order: this rank's slice goes straight into its columns of its own y
 * (iq_qmv for rows <= 16, iq_qmm for larger multiples of 64, with their preconditions and workspace); then all ranks meet
 * (none of them still reads the previous call's y), each stores its slice into the same columns of every peer's y with
 * 16-byte peer stores, and they meet again: when the call's kernels have run, y holds all n output features on every
 * rank. For one to sixteen rows the exchange is one small kernel. The waits are bounded (iq_ctx_set_wait_cycles;
 * IQ_ERR_TIMEOUT in iq_ctx_status when a peer never arrives). n a multiple of 16 * world; at most 8 ranks. With
 * IQ_FLAG_NO_BARRIER the barriers are left out and the host must order the ranks (and the reuse of y) itself. */
typedef struct iq_colsplit iq_colsplit;
int32_t iq_colsplit_create(iq_ctx* ctx, int32_t rank, int32_t world, int32_t n_total, int32_t max_rows, int32_t y_dtype,
                           void* const* peer_y, void* const* peer_flags, iq_colsplit** out);
void iq_colsplit_destroy(iq_colsplit* cs);
int32_t iq_linear_colsplit_workspace_bytes(iq_colsplit* cs, const iq_qlinear* shard, int32_t rows, int32_t x_dtype,
                                           size_t* bytes);
int32_t iq_linear_colsplit(iq_colsplit* cs, void* stream, const void* x, int32_t x_dtype, int64_t ldx,
                           const iq_qlinear* shard, int32_t rows, uint32_t flags, void* workspace, size_t workspace_bytes);

/* ---- before the first layer -------------------------------------------------------------------------------------------
 * Embedding gather: row tokens[r] of the table, dequantised as float(scale) * code + float(bias) in fp32, into out_f32
 * [rows, ldo] and / or its fp16 rounding out_f16 [rows, ldo] (either may be NULL). Replaces embed_rows, embed_rows_g32,
 * embed_rows_b6, embed_rows_b8 and embed_rows_bf16 (Shaders/yy_model.metal:12-95, Shaders/yw_lfm.metal; bit-exact check in KernelCaseG32.swift:80-93).
 * table: affine 4-bit (group 64 or 32), 6-bit or 8-bit (group 64); bits = 16 is a plain bf16 table (scales and biases
 * unused).
 * tokens is a device array; a token >= table->n gives a zero row. */
int32_t iq_embed_rows(iq_ctx* ctx, void* stream, const iq_qlinear* table, const uint32_t* tokens, int32_t rows,
                      float* out_f32, void* out_f16, int64_t ldo);

/* ---- the rotated ternary format ------------------------------------------------------------------------------------------
 * y[r, :] = half(H_1024(x[r, :] * signs) / 32) per block of 1024 inputs: the input rotation that precedes every ternary
 * matrix (had_rows_h, Shaders/xc_tern.metal:29-40; DenseQ.encodeRotate in Layers/Linear.swift:292-297). x of any
 * dtype, y fp16 [rows, ldy], k a multiple of 1024, signs fp32 [k]. iq_qmv (fp16 x, rows <= 16) and iq_qmm then take the
 * rotated rows with a 2-bit iq_qlinear. */
int32_t iq_had_rows(iq_ctx* ctx, void* stream, const void* x, int32_t x_dtype, int64_t ldx, const float* signs, void* y_f16,
                    int64_t ldy, int32_t rows, int32_t k);
/* Rows of a ternary table, dequantised and rotated back (H_1024(row) / 32 * signs): embed_rows_t
 * (Shaders/xc_tern.metal:44-65; the bonsai-embed case, Tests/IngotTests/KernelCaseTests.swift:133-155). */
int32_t iq_embed_rows_ternary(iq_ctx* ctx, void* stream, const iq_qlinear* table, const float* signs, const uint32_t* tokens,
                              int32_t rows, float* out_f32, void* out_f16, int64_t ldo);

/* ---- after the lm_head GEMV (decode) ----------------------------------------------------------------------------------
 * out[r] = index of the largest of x[r, 0..n), ties to the lower index (argmax_rows, Shaders/verify.metal:525-547). */
int32_t iq_argmax_rows(iq_ctx* ctx, void* stream, const float* x, int64_t ldx, int32_t rows, int32_t n, uint32_t* out);
/* The 64 candidates of each row of logits the sampler works on (TopK64: topk64_part + topk64_merge, zz_sample.metal;
 * contract in Tests/IngotTests/TopK64Tests.swift): idx / val [rows, 64] = the logits x >= -FLT_MAX ordered by value
 * descending, ties to the lower id, padded with (0xFFFFFFFF, -FLT_MAX); val holds the logits' own bits; z[2r] = the
 * row maximum, z[2r+1] = sum_i exp((x_i - max) / T_r). temperatures: host array of 1 value or one per row. 1..16 rows,
 * up to 262,144 logits per row. */
int32_t iq_topk64_scratch_bytes(int32_t rows, int32_t vocab, size_t* bytes);
int32_t iq_topk64(iq_ctx* ctx, void* stream, const float* x, int64_t ldx, int32_t rows, int32_t vocab,
                  const float* temperatures, int32_t n_temperatures, uint32_t* idx, float* val, float* z, void* scratch,
                  size_t scratch_bytes);

/* ---- weight loader (host only; no GPU needed) -------------------------------------------------------------------------
 * One safetensors file mapped read-only with its header parsed into a tensor table: MappedFile + the per-shard part of
 * SafetensorsStore (Loader/Safetensors.swift:46-148). `data` points into the mapping (it may be unaligned) and stays
 * valid until iq_st_close. Directory / index.json handling, per-path quantization from config.json and the assembly of
 * device layouts live in the host mirror (ingot_b200/loader.py), as they live in Swift in the reference. */
typedef enum iq_st_dtype { IQ_ST_BF16 = 0, IQ_ST_F16 = 1, IQ_ST_F32 = 2, IQ_ST_U32 = 3, IQ_ST_I32 = 4, IQ_ST_U8 = 5 } iq_st_dtype;
typedef struct iq_st iq_st;
typedef struct iq_st_tensor {
    const char* name;            /* owned by the file handle */
    int32_t dtype;               /* iq_st_dtype */
    int32_t rank;
    int64_t shape[8];
    uint64_t file_offset;        /* absolute offset in the file (header included) */
    uint64_t bytes;
    const unsigned char* data;   /* file_offset into the mapping */
} iq_st_tensor;
int32_t iq_st_open(const char* path, iq_st** out);
void iq_st_close(iq_st* file);
int32_t iq_st_count(const iq_st* file);
int32_t iq_st_entry(const iq_st* file, int32_t index, iq_st_tensor* out);
int32_t iq_st_find(const iq_st* file, const char* name, iq_st_tensor* out);
const char* iq_st_last_error(void);  /* message of the calling thread's last failed iq_st_* call */
/* Packed 4-bit words to 8-bit words with every value times 16 (source_words words in, twice as many out; src may be
 * unaligned), and the matching bf16 scales divided by 16, which is exact: a 4-bit piece concatenated with 8-bit ones
 * keeps its values bit for bit (widen4to8Words, Layers/Linear.swift:599-610, :170-175). */
void iq_widen4to8_words(const void* src, void* dst, size_t source_words);
void iq_scales_div16_bf16(const void* src, void* dst, size_t count);

/* ---- layer-stack helper ----------------------------------------------------------------------------------------------
 * out = x / sqrt(mean(x^2) + eps) per row, unit weight: the input normalisation between the fp32 residual and an FFN
 * (the reference's rmsnorm kernels, Shaders/verify.metal:503-523; used by the 48-layer benchmark stack). */
int32_t iq_rmsnorm(iq_ctx* ctx, void* stream, const float* x, int64_t ldx, void* out, int32_t out_dtype, int64_t ldo,
                   int32_t rows, int32_t d, float eps);

#ifdef __cplusplus
}
#endif
#endif /* INGOT_QMM_H */
