// Decode GEMV on the int8 tensor-core path: y[m, n] = sum_k x[m, k] * (s[n, g] * q[n, k] + b[n, g]) for up to eight
// activation rows per launch (the host cuts 9..16 rows into two launches) and affine 4-, 6- or 8-bit weights.
//
// Why integers. The fp16 formulation converts every code to a half (several ALU instructions per code) before the MMA
// and ends up bound by instruction issue at a third of the memory roofline. Here the codes go into the MMA as they
// are: 8-bit codes untouched, 4-bit codes split by two masks per 32-bit word. The activations are what gets
// converted, once per call: per group of 64 inputs they become block fixed point, X = round(x * 2^(13 - e)) with
// 2^e >= max|x| of the group, split into two signed 7-bit digits X = 128 * hi + lo. The digits are the B operand
// (m16n8k32, u8 x s8 -> s32): the eight B columns are (row, digit) pairs, so one MMA serves four rows (rows 4..7 take
// a second pair of MMAs on the same unpacked codes). A row's arithmetic does not depend on the other rows of the
// call, which is what makes its bits the same alone, among 4 and among 16. Per group the
// exact integer sums give
//     sum_k x q  ~=  2^(e - 13) * (128 * acc_hi + acc_lo)        (error <= 2^-14 of the group's largest |x| per input)
// and the group's contribution is s * that + b * sum_k x, with sum_k x kept in fp32. That is two MMAs, two integer
// and six float instructions per 64 x 16 weights, against several hundred in the fp16 formulation.
//
// Structure: persistent CTAs (two per SM up to four rows) each own a contiguous range of 16-row blocks and walk it block
// by block. Warp 8 streams each 16-row block through a ring of bulk copies (one per
// pair of rows, the pairs padded apart so that the fragment loads are free of bank conflicts, plus scales and biases;
// or one swizzled tensor copy per block where rows are short); the 8
// consumer warps take one slice of K each, and their partial sums meet in shared memory in a fixed order. Every wait is bounded.
//
// Same operator as the reference's vnax_qmv* kernels (Shaders/verify_nax.metal:105-230); taken when K is a multiple
// of 2048 and the activations of eight rows plus two stages fit shared memory (a choice that does not look at the row
// count), the fp16 kernels serve the rest.
#pragma once

#include "common.cuh"
#include "ptx.cuh"

namespace iq {

constexpr int kQiMaxThreads = 320;  // 8 consumer warps + the producer warp + the tail warp
constexpr int kQiRows = 16;         // weight rows per stage (MMA M)
constexpr int kQiPiece = 8192;      // bytes per bulk copy

struct QiParams {
    const unsigned char* w;
    const unsigned char* s;
    const unsigned char* b;
    int32_t N, K, M;
    const void* x;
    int32_t x_dtype;
    int64_t ldx;
    void* y;
    int32_t y_dtype;
    int64_t ldy;
    int32_t accumulate;
    int32_t row_bytes;    // code bytes per weight row
    int32_t row_pitch;    // the padded pitch of a row, or of a pair of rows (pair != 0), inside a stage
    int32_t pair;         // rows are staged two per bulk copy
    int32_t srow_bytes;   // scale bytes per weight row (= bias bytes)
    int32_t srow_pitch;   // ... and their padded pitch inside a stage
    int32_t stage_bytes, nstages;
    int32_t xq_bytes, xsc_bytes, red_bytes;
    int32_t ncw;          // consumer warps (8 or 16): K slices per block of rows; the producer is warp ncw
    // Tail split (tail_blocks > 0): every CTA walks blocks_per_cta whole blocks; the tail_blocks blocks left over are cut
    // into tail_slices K slices each and dealt out one piece per CTA, so that no CTA walks one block more than the rest.
    int32_t blocks_per_cta, tail_blocks, tail_slices;
    float* tail_scratch;        // [tail_blocks * tail_slices][MS][64] partial sums of the pieces
    uint32_t* tail_counters;    // [tail_blocks] pieces done; the CTA that finishes a block's last piece adds them up
    int32_t* status;
};

__device__ __forceinline__ void imma16832_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1, const int (&c)[4]) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}

// Shared-memory loads the compiler may reorder among themselves and around the MMAs (not volatile), but not hoist above
// the wait whose result is `token`: the token is an input, and it differs from item to item, so a load of one item is
// never taken for the same address's load of another.
__device__ __forceinline__ uint2 lds64_after(uint32_t addr, uint32_t token) {
    uint2 v;
    asm("ld.shared.v2.u32 {%0,%1}, [%2]; // %3" : "=r"(v.x), "=r"(v.y) : "r"(addr), "r"(token));
    return v;
}
__device__ __forceinline__ uint4 lds128_after(uint32_t addr, uint32_t token) {
    uint4 v;
    asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4]; // %5" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "r"(token));
    return v;
}
__device__ __forceinline__ uint32_t lds32_after(uint32_t addr, uint32_t token) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1]; // %2" : "=r"(v) : "r"(addr), "r"(token));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16_after(uint32_t addr, uint32_t token) {
    uint32_t v;
    asm("ld.shared.u16 %0, [%1]; // %2" : "=r"(v) : "r"(addr), "r"(token));
    return v;
}
__device__ __forceinline__ float2 lds64f_after(uint32_t addr, uint32_t token) {
    float2 v;
    asm("ld.shared.v2.f32 {%0,%1}, [%2]; // %3" : "=f"(v.x), "=f"(v.y) : "r"(addr), "r"(token));
    return v;
}

// Four 6-bit codes in the low 24 bits of v (whatever sits above them) -> one code per byte.
__device__ __forceinline__ uint32_t spread6(uint32_t v) {
    const uint32_t y = (v & 0x00000FFFu) | ((v << 4) & 0x0FFF0000u);  // twelve bits per 16-bit half
    return (y & 0x003F003Fu) | ((y << 2) & 0x3F003F00u);
}
// Sixteen 6-bit codes, a little-endian stream of 96 bits in three words, as sixteen bytes: word j holds codes 4j..4j+3.
__device__ __forceinline__ void unpack6x16(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t (&o)[4]) {
    o[0] = spread6(w0);
    o[1] = spread6(__funnelshift_r(w0, w1, 24));
    o[2] = spread6(__funnelshift_r(w1, w2, 16));
    o[3] = spread6(w2 >> 8);
}

// Block fixed point of one group of 64 activations: from the group's largest magnitude and its sum, the power of two
// 2^(e-13) the digits are counted in (2^e > amax >= 2^(e-1)) and its inverse. A group that holds a NaN or an infinity
// (amax or the sum not finite; fmaxf drops a NaN, the sum keeps it) gets a NaN scale and a NaN sum, so that every output
// it feeds comes out NaN, where the fp16 kernels and an fp32 matrix product give NaN or an infinity: a non-finite input
// must not turn into a finite output. Groups whose largest magnitude is below 2^-100 count as zero.
__device__ __forceinline__ void qi_group_scale(float amax, float& sum, float& scale, float& inv) {
    scale = 0.f;
    inv = 0.f;
    if (!(amax <= 3.4028235e38f) || !(fabsf(sum) <= 3.4028235e38f)) {
        scale = __uint_as_float(0x7FC00000u);
        sum = scale;
        return;
    }
    if (amax > 0.f) {
        const int e = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 126;
        if (e > -100) {
            scale = __uint_as_float((uint32_t)(e - 13 + 127) << 23);
            inv = __uint_as_float((uint32_t)(13 - e + 127) << 23);
        }
    }
}

// Barrier over the consumer warps; the value it returns (zero) is a token for loads that must stay behind it.
__device__ __forceinline__ uint32_t qi_consumer_barrier(int threads) {
    uint32_t t;
    asm volatile("bar.sync 1, %1;\n\tmov.u32 %0, 0;" : "=r"(t) : "r"(threads) : "memory");
    return t;
}
__device__ __forceinline__ bool qi_consumer_barrier_or(int threads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n.reg .pred p, q;\nsetp.ne.u32 p, %1, 0;\nbar.red.or.pred q, 1, %2, p;\nselp.u32 %0, 1, 0, q;\n}\n"
        : "=r"(r)
        : "r"((uint32_t)pred), "r"(threads)
        : "memory");
    return r != 0;
}

// FMT: kFmtAffine4, kFmtAffine8 or kFmtAffine6; MS: sets of four activation rows (1 or 2); GW: groups of 64 inputs per consumer warp
// when known at compile time (the activation fragments of the warp's K slice then live in registers across all row
// blocks), 0 when not.
template <int FMT, int MS, int GW, bool TM = false>
__global__ void __launch_bounds__(kQiMaxThreads, MS == 1 ? 2 : 1)
    qmv_imma_kernel(const __grid_constant__ CUtensorMap wmap, const QiParams p) {
    constexpr bool W6 = FMT == kFmtAffine6;
    // W8: one code per operand byte, lane t of a quad owns inputs 16t..16t+15 of a group (8-bit codes as they are, 6-bit
    // codes after unpacking); otherwise 4-bit codes, two per byte, split by masks
    constexpr bool W8 = FMT == kFmtAffine8 || W6;
    constexpr int GB = W6 ? 48 : (W8 ? 64 : 32);  // code bytes per group of 64 inputs
    constexpr int LB = GB / 4;                    // ... and per lane of a quad
    // TM: a block of 16 rows arrives as one tensor copy with the 128-byte swizzle, laid out [128-byte column][row][128]:
    // the byte at offset o of row r sits at (o / 128) * 2048 + r * 128 + ((o / 16 % 8) ^ (r % 8)) * 16 + o % 16, which puts
    // the eight rows a fragment load touches in eight different bank groups without padding the rows. One copy per block
    // instead of one per row: with rows of 1 KB (4-bit, K = 2048) the per-row copies' issue rate, about one per 35 ns and
    // SM, bounds the kernel at 0.6 of the memory roofline, the tensor copy reaches 0.8. With rows of 2 KB and more the
    // per-row copies already run at the memory's rate and start faster, so they stay.
    // Not TM: one bulk copy per row into padded rows, or (p.pair) per pair of neighbouring rows, which are one stretch of
    // memory, the pairs padded apart and the MMA's rows g and g + 8 the two rows of pair g. Pairs measured faster for
    // 6- and 8-bit rows (44.2 against 47.7 us on a 128000 x 2048 6-bit head), single rows for 4-bit rows of 2 KB (9.0
    // against 9.6 us on 14336 x 4096, where the first block's arrival counts for more than the copies' number).
    static_assert(!TM || FMT == kFmtAffine4, "tensor-copy staging is built for 4-bit codes");
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char* xq = smem;                                            // [groups][MS][32 lanes] uint4: B fragments
    float2* xsc = reinterpret_cast<float2*>(smem + p.xq_bytes);          // [groups][MS * 4 rows] {2^(e-13), sum x}
    float* red = reinterpret_cast<float*>(smem + p.xq_bytes + p.xsc_bytes);  // [2][consumer warps][MS][32 lanes][2]
    unsigned char* stages = smem + p.xq_bytes + p.xsc_bytes + p.red_bytes;
    if (TM) stages += (1024u - (smem_u32(stages) & 1023u)) & 1023u;  // the swizzle pattern is a function of the address
    const int ncw = p.ncw, nct = 32 * p.ncw;  // consumer warps and threads
    uint64_t* bars = reinterpret_cast<uint64_t*>(stages + (size_t)p.nstages * p.stage_bytes);
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * p.nstages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * p.nstages);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (TM && tid == 32 * p.ncw)  // the descriptor's fetch starts now, not with the first copy
        asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
    if (tid == 0) {
        for (int s = 0; s < p.nstages; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, ncw);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    __syncthreads();
    pdl_launch_dependents();

    // This CTA's rows: a contiguous range of whole 16-row blocks (the last block of the matrix may be short). Cutting the
    // range at arbitrary rows would balance the bytes better, but a block with one row costs the instructions of a full
    // one, and the kernel is bound by instruction issue before it is bound by bytes.
    const int nblk = (p.N + kQiRows - 1) / kQiRows;
    int lo, hi;
    if (p.tail_blocks > 0) {
        lo = blockIdx.x * p.blocks_per_cta * kQiRows;
        hi = lo + p.blocks_per_cta * kQiRows;
    } else {
        lo = (int)((int64_t)nblk * blockIdx.x / gridDim.x) * kQiRows;
        hi = min(p.N, (int)((int64_t)nblk * (blockIdx.x + 1) / gridDim.x) * kQiRows);
    }
    const int items = (hi - lo + kQiRows - 1) / kQiRows;
    const int G = p.K / 64;
    const bool pair = !TM && p.pair != 0;
    const int codes_bytes = TM ? kQiRows * p.row_bytes : (pair ? kQiRows / 2 : kQiRows) * p.row_pitch;
    const int sc_bytes = kQiRows * p.srow_pitch;

    // ---- tail pieces: (left-over block, K slice), one warp per piece, weights straight from global memory. Run by a
    // warp of its own beside the row blocks, so that the pieces' latencies (global loads, fence, counter) cost them nothing.
    const int g = lane >> 2, t = lane & 3;
    const uint32_t xq32 = smem_u32(xq) + lane * 16, xsc32 = smem_u32(xsc) + t * 8;
    auto tail_pieces = [&](uint32_t xtok) {
        const int gp = G / p.tail_slices;  // groups per piece
        const int base_rows = (int)gridDim.x * p.blocks_per_cta * kQiRows;
        for (int pc = blockIdx.x; pc < p.tail_blocks * p.tail_slices; pc += gridDim.x) {
            const int tb = pc / p.tail_slices, sl = pc % p.tail_slices;
            const int r0 = base_rows + tb * kQiRows;
            const unsigned char* w0p = p.w + (size_t)(r0 + g) * p.row_bytes + t * LB;
            const unsigned char* w1p = w0p + (size_t)8 * p.row_bytes;
            const uint16_t* s0p = reinterpret_cast<const uint16_t*>(p.s + (size_t)(r0 + g) * p.srow_bytes);
            const uint16_t* s1p = reinterpret_cast<const uint16_t*>(p.s + (size_t)(r0 + g + 8) * p.srow_bytes);
            const uint16_t* b0p = reinterpret_cast<const uint16_t*>(p.b + (size_t)(r0 + g) * p.srow_bytes);
            const uint16_t* b1p = reinterpret_cast<const uint16_t*>(p.b + (size_t)(r0 + g + 8) * p.srow_bytes);
            float a0[MS], a1[MS];
#pragma unroll
            for (int c = 0; c < MS; c++) a0[c] = a1[c] = 0.f;
            for (int grp = sl * gp; grp < (sl + 1) * gp; grp++) {
                const int z[4] = {0, 0, 0, 0};
                uint32_t a[2][4];
                if (W6) {
                    const uint32_t* q0 = reinterpret_cast<const uint32_t*>(w0p + grp * GB);
                    const uint32_t* q1 = reinterpret_cast<const uint32_t*>(w1p + grp * GB);
                    uint32_t o0[4], o1[4];
                    unpack6x16(__ldg(q0), __ldg(q0 + 1), __ldg(q0 + 2), o0);
                    unpack6x16(__ldg(q1), __ldg(q1 + 1), __ldg(q1 + 2), o1);
                    a[0][0] = o0[0]; a[0][1] = o1[0]; a[0][2] = o0[1]; a[0][3] = o1[1];
                    a[1][0] = o0[2]; a[1][1] = o1[2]; a[1][2] = o0[3]; a[1][3] = o1[3];
                } else if (W8) {
                    const uint4 w0 = ldg_nc_u4(w0p + grp * GB), w1 = ldg_nc_u4(w1p + grp * GB);
                    a[0][0] = w0.x; a[0][1] = w1.x; a[0][2] = w0.y; a[0][3] = w1.y;
                    a[1][0] = w0.z; a[1][1] = w1.z; a[1][2] = w0.w; a[1][3] = w1.w;
                } else {
                    const uint2 w0 = *reinterpret_cast<const uint2*>(w0p + grp * GB);
                    const uint2 w1 = *reinterpret_cast<const uint2*>(w1p + grp * GB);
                    constexpr uint32_t MSK = 0x0F0F0F0Fu;
                    a[0][0] = w0.x & MSK; a[0][1] = w1.x & MSK; a[0][2] = (w0.x >> 4) & MSK; a[0][3] = (w1.x >> 4) & MSK;
                    a[1][0] = w0.y & MSK; a[1][1] = w1.y & MSK; a[1][2] = (w0.y >> 4) & MSK; a[1][3] = (w1.y >> 4) & MSK;
                }
                const float sc0 = bf16_bits_to_f32(s0p[grp]), sc1 = bf16_bits_to_f32(s1p[grp]);
                const float bi0 = bf16_bits_to_f32(b0p[grp]), bi1 = bf16_bits_to_f32(b1p[grp]);
#pragma unroll
                for (int c = 0; c < MS; c++) {
                    int d[4];
                    const uint4 xb = lds128_after(xq32 + (grp * MS + c) * 512, xtok);
                    imma16832_u8s8(d, a[0][0], a[0][1], a[0][2], a[0][3], xb.x, xb.y, z);
                    imma16832_u8s8(d, a[1][0], a[1][1], a[1][2], a[1][3], xb.z, xb.w, d);
                    const float2 xs = lds64f_after(xsc32 + (grp * MS + c) * 32, xtok);
                    const float v0 = (float)(d[0] * 128 + d[1]), v1 = (float)(d[2] * 128 + d[3]);
                    a0[c] = fmaf(v0, sc0 * xs.x, a0[c]);
                    a0[c] = fmaf(bi0, xs.y, a0[c]);
                    a1[c] = fmaf(v1, sc1 * xs.x, a1[c]);
                    a1[c] = fmaf(bi1, xs.y, a1[c]);
                }
            }
            float* part = p.tail_scratch + (size_t)pc * (MS * 64);
#pragma unroll
            for (int c = 0; c < MS; c++) {
                __stcg(part + c * 64 + lane * 2, a0[c]);
                __stcg(part + c * 64 + lane * 2 + 1, a1[c]);
            }
            __threadfence();
            __syncwarp();
            uint32_t done = 0;
            if (lane == 0) done = atomicAdd(p.tail_counters + tb, 1u);
            done = __shfl_sync(0xffffffffu, done, 0);
            if (done != (uint32_t)p.tail_slices - 1) continue;
            // this warp finished the block's last piece: add the slices up in slice order and store
            __threadfence();
#pragma unroll
            for (int c = 0; c < MS; c++) {
                const int m = 4 * c + t;
                float y0 = 0.f, y1 = 0.f;
                for (int k = 0; k < p.tail_slices; k++) {
                    const float* q = p.tail_scratch + (size_t)(tb * p.tail_slices + k) * (MS * 64) + c * 64 + lane * 2;
                    y0 += __ldcg(q);
                    y1 += __ldcg(q + 1);
                }
                if (m >= p.M) continue;
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const float v = h ? y1 : y0;
                    const size_t o = (size_t)m * p.ldy + r0 + g + 8 * h;
                    if (p.y_dtype == kF32) {
                        float* yp = reinterpret_cast<float*>(p.y) + o;
                        *yp = p.accumulate ? *yp + v : v;
                    } else if (p.y_dtype == kF16) {
                        __half* yp = reinterpret_cast<__half*>(p.y) + o;
                        *yp = __float2half_rn(p.accumulate ? __half2float(*yp) + v : v);
                    } else {
                        uint16_t* yp = reinterpret_cast<uint16_t*>(p.y) + o;
                        *yp = (uint16_t)f32_to_bf16_bits(p.accumulate ? bf16_bits_to_f32(*yp) + v : v);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) atomicExch(p.tail_counters + tb, 0u);  // ready for the slot's next launch
        }
    };

    if (warp == ncw) {
        // ================= producer: weights do not depend on the previous kernel, so it starts at once =========
        bool ok = true;
        for (int it = 0; it < items && ok; it++) {
            const int s = it % p.nstages;
            const uint32_t ph = (it / p.nstages) & 1;
            const int r0 = lo + it * kQiRows;
            const int rows = min(kQiRows, hi - r0);
            ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            // (a tensor copy counts its whole box, rows beyond the matrix arrive as zeros)
            if (lane == 0)
                mbar_arrive_expect_tx(bar_full + 8 * s, (TM ? kQiRows : rows) * p.row_bytes + rows * 2 * p.srow_bytes);
            __syncwarp();
            const uint32_t st = smem_u32(stages + (size_t)s * p.stage_bytes);
            if (TM) {
                if (lane == 0) tma_load_3d(st, &wmap, bar_full + 8 * s, 0, r0, 0);
            } else if (pair) {
                if (2 * lane < rows) {  // lanes 0-7: the codes of two neighbouring rows each, one stretch of memory
                    const unsigned char* src = p.w + (size_t)(r0 + 2 * lane) * p.row_bytes;
                    const int bytes = min(2, rows - 2 * lane) * p.row_bytes;
                    for (int off = 0; off < bytes; off += kQiPiece)
                        bulk_g2s(st + lane * p.row_pitch + off, src + off, min(kQiPiece, bytes - off), bar_full + 8 * s);
                }
            } else if ((lane & 15) < rows) {
                // lanes 0-15: the first half of one row each, lanes 16-31: the second half (32 copies in flight at once
                // bring a 2 KB-row block in sooner than 16: 8.80 against 8.95 us on 14336 x 4096)
                const int hb = p.row_bytes >> 1, o0 = (lane >> 4) * hb;
                const unsigned char* src = p.w + (size_t)(r0 + (lane & 15)) * p.row_bytes + o0;
                for (int off = 0; off < hb; off += kQiPiece)
                    bulk_g2s(st + (lane & 15) * p.row_pitch + o0 + off, src + off, min(kQiPiece, hb - off), bar_full + 8 * s);
            }
            if (lane == 16) {
                bulk_g2s(st + codes_bytes, p.s + (size_t)r0 * p.srow_bytes, rows * p.srow_bytes, bar_full + 8 * s);
            } else if (lane == 17) {
                bulk_g2s(st + codes_bytes + sc_bytes, p.b + (size_t)r0 * p.srow_bytes, rows * p.srow_bytes, bar_full + 8 * s);
            }
        }
        if (!ok) {  // give copies in flight time to land before the CTA's shared memory is released
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {}
        }
    } else if (warp == ncw + 1) {
        // ================= tail warp: the left-over blocks' pieces, beside the row blocks =================
        if (p.tail_blocks > 0) {
            uint32_t tk;
            pdl_wait();  // y belongs to the previous kernel until here
            asm volatile("bar.sync 2, %1;\n\tmov.u32 %0, 0;" : "=r"(tk) : "r"(nct + 32) : "memory");  // xq is ready
            tail_pieces(tk);
        }
    } else {
        // ================= consumers =================
        pdl_wait();  // the activations (and y) belong to the previous kernel until here
        // ---- activations -> block fixed point, two 7-bit digits, in B-fragment order --------------------------------
        // One thread per eight consecutive inputs (the span of one 32-bit word of 4-bit codes); the eight threads of a
        // group find its largest magnitude and its sum with a fixed shuffle tree, so a row's digits and sums do not
        // depend on the other rows.
        // rows the call does not have: zero digits, zero scale
        for (int u = tid; u < G * 8 * (4 * MS - p.M); u += nct) {
            const int m = p.M + u / (G * 8), j = (u >> 3) % G, w8 = u & 7;
            const int fb = ((j * MS + (m >> 2)) * 32 + 8 * (m & 3)) * 16 + (w8 & 1) * 8 + (w8 >> 1) * 16;
            *reinterpret_cast<uint2*>(xq + fb) = make_uint2(0, 0);
            *reinterpret_cast<uint2*>(xq + fb + 64) = make_uint2(0, 0);
            if (w8 == 0) xsc[j * 4 * MS + m] = make_float2(0.f, 0.f);
        }
        for (int u = tid; u < G * 8 * p.M; u += nct) {
            const int m = u / (G * 8), j = (u >> 3) % G, w8 = u & 7;
            float v[8];
            load_x8(p.x, p.x_dtype, (size_t)m * p.ldx + j * 64 + w8 * 8, v);
            float amax = 0.f, sum = 0.f;
#pragma unroll
            for (int k = 0; k < 8; k++) {
                amax = fmaxf(amax, fabsf(v[k]));
                sum += v[k];
            }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                sum += __shfl_xor_sync(0xffffffffu, sum, o);
            }
            float scale, inv;
            qi_group_scale(amax, sum, scale, inv);
            if (w8 == 0) xsc[j * 4 * MS + m] = make_float2(scale, sum);
            uint32_t hi_w[2] = {0, 0}, lo_w[2] = {0, 0};  // [b0 / b1 half] bytes i = 0..3
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int X = __float2int_rn(v[k] * inv);       // |X| <= 8192
                const int hi_d = (X + 64) >> 7, lo_d = X - (hi_d << 7);
                // input k of the span: 4-bit codes put even k in the low nibbles (b0) and odd k in the high ones (b1);
                // 8-bit codes put k 0-3 in one word (b0) and k 4-7 in the next (b1)
                const int half = W8 ? (k >> 2) : (k & 1), i = W8 ? (k & 3) : (k >> 1);
                hi_w[half] |= (uint32_t)(hi_d & 0xFF) << (8 * i);
                lo_w[half] |= (uint32_t)(lo_d & 0xFF) << (8 * i);
            }
            // the span is word w8 of the group's eight (4-bit: lane t = w8 / 2, MMA w8 % 2) or words 2 w8, 2 w8 + 1 of
            // its sixteen (8-bit: lane t = w8 / 2, MMA w8 % 2): the same slot either way
            const int t = w8 >> 1, mm = w8 & 1;
            const int fb = ((j * MS + (m >> 2)) * 32 + 8 * (m & 3)) * 16 + mm * 8;  // the row's hi-digit column, lane 0
            *reinterpret_cast<uint2*>(xq + fb + t * 16) = make_uint2(hi_w[0], hi_w[1]);
            *reinterpret_cast<uint2*>(xq + fb + (4 + t) * 16) = make_uint2(lo_w[0], lo_w[1]);
        }
        const uint32_t xtok = qi_consumer_barrier(nct);
        if (p.tail_blocks > 0) asm volatile("bar.arrive 2, %0;" ::"r"(nct + 32) : "memory");  // the producer may read xq

        const int gw = GW > 0 ? GW : G / ncw;       // groups per warp (a multiple of 4)
        const int g0 = warp * gw;
        uint4 xbr[GW > 0 ? GW : 1][MS];
        float2 xsr[GW > 0 ? GW : 1][MS];
        if (GW > 0) {
#pragma unroll
            for (int q = 0; q < GW; q++)
#pragma unroll
                for (int c = 0; c < MS; c++) {
                    xbr[q][c] = lds128_after(xq32 + ((g0 + q) * MS + c) * 512, xtok);
                    xsr[q][c] = lds64f_after(xsc32 + ((g0 + q) * MS + c) * 32, xtok);
                }
        }
        // TM: where the lane's piece of group q of a run of four groups sits, relative to row g of the run's first column
        uint32_t xo[4];
#pragma unroll
        for (int q = 0; q < 4; q++) xo[q] = (((2 * q + (t >> 1)) ^ g) << 4) + ((t & 1) << 3);
        for (int it = 0; it < items; it++) {
            const int s = it % p.nstages;
            const uint32_t ph = (it / p.nstages) & 1;
            const int r0 = lo + it * kQiRows;
            const int rows = min(kQiRows, hi - r0);
            const bool ok = mbar_wait(bar_full + 8 * s, ph, abort_flag);
            const uint32_t tok = (uint32_t)it + (ok ? 0u : 0x80000000u);  // orders the stage's loads after the wait
            float acc0[MS], acc1[MS];  // rows g and g + 8 of the block, activation rows t, 4 + t
#pragma unroll
            for (int c = 0; c < MS; c++) acc0[c] = acc1[c] = 0.f;
            if (ok) {
                const uint32_t st = smem_u32(stages + (size_t)s * p.stage_bytes);
                // not TM: row g of the padded stage, the lane's piece of group 0. TM: row g of the first 128-byte column
                // this warp reads (four 4-bit groups per column); xo[] adds the swizzled piece.
                // Pairs: MMA rows g and g + 8 are the two rows of pair g (rows 2g and 2g + 1 of the block), which arrived as
                // one copy; rows or pairs are padded apart so that the eight a load touches sit in different banks.
                const uint32_t wa0 = TM ? st + g * 128 + (g0 >> 2) * 2048 : st + g * p.row_pitch + t * LB;
                const uint32_t wa1 = wa0 + (TM ? 1024 : (pair ? p.row_bytes : 8 * p.row_pitch));
                const uint32_t sa0 = st + codes_bytes + (pair ? 2 * g : g) * p.srow_pitch;
                const uint32_t sa1 = sa0 + (pair ? 1 : 8) * p.srow_pitch;
#pragma unroll
                for (int c4 = 0; c4 < (GW > 0 ? GW : gw); c4 += 4) {
                    // scales and biases of four groups for both rows (bf16 pairs)
                    const uint2 s0 = lds64_after(sa0 + (g0 + c4) * 2, tok), s1 = lds64_after(sa1 + (g0 + c4) * 2, tok);
                    const uint2 b0 = lds64_after(sa0 + sc_bytes + (g0 + c4) * 2, tok);
                    const uint2 b1 = lds64_after(sa1 + sc_bytes + (g0 + c4) * 2, tok);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int grp = g0 + c4 + q;
                        const int z[4] = {0, 0, 0, 0};
                        uint32_t a[2][4];  // the A fragments of the group's two MMAs
                        if (W6) {
                            uint32_t o0[4], o1[4];
                            const uint32_t q0 = wa0 + grp * GB, q1 = wa1 + grp * GB;
                            unpack6x16(lds32_after(q0, tok), lds32_after(q0 + 4, tok), lds32_after(q0 + 8, tok), o0);
                            unpack6x16(lds32_after(q1, tok), lds32_after(q1 + 4, tok), lds32_after(q1 + 8, tok), o1);
                            a[0][0] = o0[0]; a[0][1] = o1[0]; a[0][2] = o0[1]; a[0][3] = o1[1];
                            a[1][0] = o0[2]; a[1][1] = o1[2]; a[1][2] = o0[3]; a[1][3] = o1[3];
                        } else if (W8) {
                            const uint4 w0 = lds128_after(wa0 + grp * GB, tok), w1 = lds128_after(wa1 + grp * GB, tok);
                            a[0][0] = w0.x; a[0][1] = w1.x; a[0][2] = w0.y; a[0][3] = w1.y;
                            a[1][0] = w0.z; a[1][1] = w1.z; a[1][2] = w0.w; a[1][3] = w1.w;
                        } else {
                            const uint32_t o = TM ? c4 * 512 + xo[q] : grp * GB;
                            const uint2 w0 = lds64_after(wa0 + o, tok), w1 = lds64_after(wa1 + o, tok);
                            constexpr uint32_t MSK = 0x0F0F0F0Fu;
                            a[0][0] = w0.x & MSK; a[0][1] = w1.x & MSK; a[0][2] = (w0.x >> 4) & MSK; a[0][3] = (w1.x >> 4) & MSK;
                            a[1][0] = w0.y & MSK; a[1][1] = w1.y & MSK; a[1][2] = (w0.y >> 4) & MSK; a[1][3] = (w1.y >> 4) & MSK;
                        }
                        const uint32_t sw0 = q < 2 ? s0.x : s0.y, sw1 = q < 2 ? s1.x : s1.y;
                        const uint32_t bw0 = q < 2 ? b0.x : b0.y, bw1 = q < 2 ? b1.x : b1.y;
                        const float sc0 = __uint_as_float((q & 1) ? (sw0 & 0xFFFF0000u) : (sw0 << 16));
                        const float sc1 = __uint_as_float((q & 1) ? (sw1 & 0xFFFF0000u) : (sw1 << 16));
                        const float bi0 = __uint_as_float((q & 1) ? (bw0 & 0xFFFF0000u) : (bw0 << 16));
                        const float bi1 = __uint_as_float((q & 1) ? (bw1 & 0xFFFF0000u) : (bw1 << 16));
#pragma unroll
                        for (int c = 0; c < MS; c++) {
                            int d[4];
                            const uint4 xb = GW > 0 ? xbr[GW > 0 ? c4 + q : 0][c] : lds128_after(xq32 + (grp * MS + c) * 512, xtok);
                            imma16832_u8s8(d, a[0][0], a[0][1], a[0][2], a[0][3], xb.x, xb.y, z);
                            imma16832_u8s8(d, a[1][0], a[1][1], a[1][2], a[1][3], xb.z, xb.w, d);
                            // {2^(e-13), sum x} of activation row 4c + t
                            const float2 xs = GW > 0 ? xsr[GW > 0 ? c4 + q : 0][c] : lds64f_after(xsc32 + (grp * MS + c) * 32, xtok);
                            const float v0 = (float)(d[0] * 128 + d[1]), v1 = (float)(d[2] * 128 + d[3]);
                            acc0[c] = fmaf(v0, sc0 * xs.x, acc0[c]);
                            acc0[c] = fmaf(bi0, xs.y, acc0[c]);
                            acc1[c] = fmaf(v1, sc1 * xs.x, acc1[c]);
                            acc1[c] = fmaf(bi1, xs.y, acc1[c]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(bar_empty + 8 * s);  // the stage is free once every warp has read its part

            // ---- the eight K slices meet in shared memory -----------------------------------------------------------------
            float* mine = red + ((it & 1) * ncw + warp) * (64 * MS);
#pragma unroll
            for (int c = 0; c < MS; c++) {
                mine[c * 64 + lane * 2] = acc0[c];
                mine[c * 64 + lane * 2 + 1] = acc1[c];
            }
            if (qi_consumer_barrier_or(nct, !ok)) break;  // a wait gave up somewhere: everybody leaves together
            // The block's 64 * MS sums, one per thread of the first 2 * MS warps, slices added in slice order; consecutive
            // lanes take consecutive weight rows, so a row of y is written 64 bytes at a time.
            if (tid >= 64 * MS) continue;
            {
                const int c = tid >> 6, mm = (tid >> 4) & 3, r = tid & 15;
                const int m = 4 * c + mm;
                if (m >= p.M || r >= rows) continue;
                // row r of the block is MMA row r / 2, half r % 2 (row pairs) or MMA row r % 8, half r / 8
                const int slot = pair ? c * 64 + (4 * (r >> 1) + mm) * 2 + (r & 1) : c * 64 + (4 * (r & 7) + mm) * 2 + (r >> 3);
                float v = 0.f;
                for (int k = 0; k < ncw; k++) v += red[((it & 1) * ncw + k) * (64 * MS) + slot];
                const size_t o = (size_t)m * p.ldy + r0 + r;
                if (p.y_dtype == kF32) {
                    float* yp = reinterpret_cast<float*>(p.y) + o;
                    *yp = p.accumulate ? *yp + v : v;
                } else if (p.y_dtype == kF16) {
                    __half* yp = reinterpret_cast<__half*>(p.y) + o;
                    *yp = __float2half_rn(p.accumulate ? __half2float(*yp) + v : v);
                } else {
                    uint16_t* yp = reinterpret_cast<uint16_t*>(p.y) + o;
                    *yp = (uint16_t)f32_to_bf16_bits(p.accumulate ? bf16_bits_to_f32(*yp) + v : v);
                }
            }
        }
    }
    __syncthreads();
    if (*abort_flag && tid == 0 && p.status != nullptr) atomicExch(p.status, kErrTimeout);
}

}  // namespace iq
