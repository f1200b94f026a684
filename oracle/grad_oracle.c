/*
 * CPU oracle for the compressed data-parallel gradient path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker, never the product:
 * only the test-suite, the smoke check and the benchmark's CPU-baseline leg
 * may load it.  The shipped library never links, loads or calls it.
 *
 * It restates, in plain C, the arithmetic of the reference project
 * (takosama/NNtrain) for this path.  Each function cites the reference file
 * and lines whose behaviour it follows.  Build with
 *     gcc -O2 -fno-fast-math -ffp-contract=off -fopenmp -shared -fPIC
 * so that every binary32 operation is one IEEE-754 round-to-nearest-even
 * operation, with no fused multiply-add and no flush-to-zero.
 *
 * Parity pinning: the reference's CPU codec is C# and cannot run where this
 * file is built, so the oracle is pinned two ways: (1) against the
 * known-answer assertions of the reference's own unit tests (zero blocks,
 * tensor-wide scale count, 128-value Mix8_32 blocks, closed-form vectors),
 * and (2) against outputs of the reference's own CUDA kernels, compiled
 * unmodified and run on a GPU, recorded as fixtures in tests/golden/.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <float.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_OK 0
#define ORACLE_ERR_ARGUMENT 1      /* bad pointer / length / block size */
#define ORACLE_ERR_NON_FINITE 2    /* reference codec throws on NaN / Inf input */
#define ORACLE_ERR_BAD_SCALE 3     /* reference storage rejects scale <= 0 or non-finite */

static inline uint32_t f32_bits(float v) { uint32_t b; memcpy(&b, &v, 4); return b; }
static inline float bits_f32(uint32_t b) { float v; memcpy(&v, &b, 4); return v; }

static int g_threads = 1;

/* Number of worker threads for the loops below (1 = the reference's own
 * single-threaded scalar loop). */
void oracle_set_threads(int threads) {
    g_threads = threads < 1 ? 1 : threads;
#ifdef _OPENMP
    omp_set_num_threads(g_threads);
#endif
}

int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}

/* Effective block size and scale count.
 * NNtrain.Core/Tensors/Bfp8Quantization.cs:64-78 (GetEffectiveBlockSize,
 * GetScaleCount): tensor-wide means one block of max(1, length) values. */
static int64_t effective_block(int64_t length, int64_t block) {
    if (block <= 0 || block >= length) return length > 0 ? length : 1;
    return block;
}

int64_t oracle_bfp8_scale_count(int64_t length, int64_t block) {
    int64_t eb = effective_block(length, block);
    return (length + eb - 1) / eb;
}

/* .NET `(int)float` is saturating and maps NaN to 0 (same as CUDA's
 * __float2int_rn); the codec then clamps to +-127.
 * NNtrain.Core/Tensors/Bfp8Quantization.cs:220-227. */
static inline int8_t code_from_quotient(float quotient) {
    float rounded = nearbyintf(quotient);   /* MathF.Round(x, ToEven) */
    int code;
    if (rounded != rounded) code = 0;
    else if (rounded >= 127.0f) code = 127;
    else if (rounded <= -127.0f) code = -127;
    else code = (int)rounded;
    return (int8_t)code;
}

/* fmaxf as used by both the C# loop (MathF.Max on finite inputs) and the
 * CUDA kernels (fmaxf drops a NaN operand). */
static inline float max_ignore_nan(float a, float b) {
    if (b != b) return a;
    return a > b ? a : b;
}

/*
 * Encode: SymmetricBfp8QuantizationCodec.Encode,
 * NNtrain.Core/Tensors/Bfp8Quantization.cs:188-236.
 *   scale = max == 0 ? 1 : max / 127   (one binary32 division)
 *   code  = clamp(round_half_even(x / scale), -127, 127)
 * strict != 0: return ORACLE_ERR_NON_FINITE on NaN/Inf input (the C# codec
 *   throws) and ORACLE_ERR_BAD_SCALE when max/127 underflows to zero (the
 *   encoded-storage constructor rejects it, :120-127).  Outputs are still
 *   written with device semantics in that case.
 * strict == 0: device semantics of the generic CUDA codec
 *   (NNtrain.Cuda/native/cuda_runtime_bridge.cu:138-192): NaN is ignored by
 *   the maximum, a NaN quotient encodes to 0, an infinite one saturates.
 */
int oracle_bfp8_encode(const float* source, int64_t length, int64_t block,
                       int8_t* payload, float* scales, int strict) {
    if (!source || !payload || !scales || length <= 0) return ORACLE_ERR_ARGUMENT;
    const int64_t eb = effective_block(length, block);
    const int64_t count = (length + eb - 1) / eb;
    int status = ORACLE_OK;
    if (count == 1) {
        /* Tensor-wide: parallelise inside the single block. */
        float maximum = 0.0f;
        int non_finite = 0;
        #pragma omp parallel for reduction(max:maximum) reduction(|:non_finite) schedule(static)
        for (int64_t i = 0; i < length; ++i) {
            float v = source[i];
            if (!isfinite(v)) non_finite = 1;
            float a = fabsf(v);
            if (a == a && a > maximum) maximum = a;
        }
        float scale = maximum == 0.0f ? 1.0f : maximum / 127.0f;
        scales[0] = scale;
        #pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < length; ++i)
            payload[i] = code_from_quotient(source[i] / scale);
        if (non_finite) status = ORACLE_ERR_NON_FINITE;
        else if (!(scale > 0.0f) || !isfinite(scale)) status = ORACLE_ERR_BAD_SCALE;
        return strict ? status : ORACLE_OK;
    }
    int any_non_finite = 0, any_bad_scale = 0;
    #pragma omp parallel for reduction(|:any_non_finite) reduction(|:any_bad_scale) schedule(static)
    for (int64_t b = 0; b < count; ++b) {
        const int64_t start = b * eb;
        const int64_t end = start + eb < length ? start + eb : length;
        float maximum = 0.0f;
        for (int64_t i = start; i < end; ++i) {
            float v = source[i];
            if (!isfinite(v)) any_non_finite = 1;
            maximum = max_ignore_nan(maximum, fabsf(v));
        }
        float scale = maximum == 0.0f ? 1.0f : maximum / 127.0f;
        scales[b] = scale;
        if (!(scale > 0.0f) || !isfinite(scale)) any_bad_scale = 1;
        for (int64_t i = start; i < end; ++i)
            payload[i] = code_from_quotient(source[i] / scale);
    }
    if (any_non_finite) status = ORACLE_ERR_NON_FINITE;
    else if (any_bad_scale) status = ORACLE_ERR_BAD_SCALE;
    return strict ? status : ORACLE_OK;
}

/*
 * Decode: SymmetricBfp8QuantizationCodec.Decode,
 * NNtrain.Core/Tensors/Bfp8Quantization.cs:238-274: x = payload * scale, one
 * binary32 multiply.  strict != 0 rejects a scale that is not finite and
 * positive (:257-262).
 */
int oracle_bfp8_decode(const int8_t* payload, const float* scales, int64_t length,
                       int64_t block, float* destination, int strict) {
    if (!payload || !scales || !destination || length <= 0) return ORACLE_ERR_ARGUMENT;
    const int64_t eb = effective_block(length, block);
    const int64_t count = (length + eb - 1) / eb;
    int bad = 0;
    for (int64_t b = 0; b < count; ++b)
        if (!isfinite(scales[b]) || !(scales[b] > 0.0f)) bad = 1;
    if (bad && strict) return ORACLE_ERR_BAD_SCALE;
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < length; ++i)
        destination[i] = (float)payload[i] * scales[i / eb];
    return ORACLE_OK;
}

/*
 * N-rank reduce of encoded gradients into fp32.
 *   r_i = s * (((x0_i + x1_i) + x2_i) + ...)   ranks in ascending order,
 *   x_k = fl(payload_k * scale_k), every add and the final multiply rounded
 *   to binary32 separately.
 * For two ranks this is the reference tests' own expectation
 * Encode(Decode(Encode a) + Decode(Encode b))
 * (NNtrain.Core.Tests/CudaBfp8GradientReducerTests.cs:44-51,
 *  CudaBfp8GradientClipNormTests.cs:249-259) with the native export's
 * reduction_scale applied to the finished sum
 * (NNtrain.Cuda/native/tensor_kernels.cu:1098-1100).  More than two ranks is
 * an extension the reference does not have (its reducers take exactly two
 * devices).
 * non_finite_out (optional) is set to 1 when any input scale is not finite
 * and positive or any r_i is not finite (tensor_kernels.cu:1092-1104).
 */
int oracle_bfp8_reduce(const int8_t* const* payloads, const float* const* scales,
                       int ranks, int64_t length, int64_t block,
                       float reduction_scale, float* reduced, int* non_finite_out) {
    if (!payloads || !scales || !reduced || ranks < 1 || length <= 0)
        return ORACLE_ERR_ARGUMENT;
    const int64_t eb = effective_block(length, block);
    const int64_t count = (length + eb - 1) / eb;
    int non_finite = 0;
    for (int r = 0; r < ranks; ++r)
        for (int64_t b = 0; b < count; ++b)
            if (!isfinite(scales[r][b]) || !(scales[r][b] > 0.0f)) non_finite = 1;
    #pragma omp parallel for reduction(|:non_finite) schedule(static)
    for (int64_t i = 0; i < length; ++i) {
        const int64_t b = i / eb;
        float sum = (float)payloads[0][i] * scales[0][b];
        for (int r = 1; r < ranks; ++r) {
            float term = (float)payloads[r][i] * scales[r][b];
            sum = sum + term;
        }
        float value = reduction_scale * sum;
        if (!isfinite(value)) non_finite = 1;
        reduced[i] = value;
    }
    if (non_finite_out) *non_finite_out = non_finite;
    return ORACLE_OK;
}

/*
 * Block transport sum (the mix8_32 bucket path): both replicas keep the raw
 * fp32 sum, no re-encode.  value = fl(fl(q0*s0) + fl(q1*s1)), extended to N
 * ranks left to right.  NNtrain.Cuda/native/gradient_collectives.cu:92-129.
 * A NaN scale (non-finite source block, :49-58) propagates into the sum.
 * squared_sum (optional) += sum of (double)value * value (:115-116).
 */
int oracle_block_transport_sum(const int8_t* const* payloads, const float* const* scales,
                               int ranks, int64_t length, int64_t block,
                               float* reduced, double* squared_sum) {
    if (!payloads || !scales || !reduced || ranks < 1 || length <= 0 || block <= 0)
        return ORACLE_ERR_ARGUMENT;
    double total = 0.0;
    #pragma omp parallel for reduction(+:total) schedule(static)
    for (int64_t i = 0; i < length; ++i) {
        const int64_t b = i / block;
        float sum = (float)payloads[0][i] * scales[0][b];
        for (int r = 1; r < ranks; ++r)
            sum = sum + (float)payloads[r][i] * scales[r][b];
        reduced[i] = sum;
        total += (double)sum * (double)sum;
    }
    if (squared_sum) *squared_sum += total;
    return ORACLE_OK;
}

/*
 * Bucket pack for the block transport: like Encode, except that a block
 * holding any NaN/Inf gets the scale bit pattern 0x7fffffff and an all-zero
 * payload.  NNtrain.Cuda/native/gradient_collectives.cu:24-60.
 */
int oracle_pack_bfp8_block(const float* source, int64_t length, int64_t block,
                           int8_t* payload, float* scales) {
    if (!source || !payload || !scales || length <= 0 || block <= 0)
        return ORACLE_ERR_ARGUMENT;
    const int64_t count = (length + block - 1) / block;
    #pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < count; ++b) {
        const int64_t start = b * block;
        const int64_t end = start + block < length ? start + block : length;
        float maximum = 0.0f;
        int non_finite = 0;
        for (int64_t i = start; i < end; ++i) {
            float v = source[i];
            if (!isfinite(v)) non_finite = 1;
            else maximum = max_ignore_nan(maximum, fabsf(v));
        }
        if (non_finite) {
            scales[b] = bits_f32(0x7fffffffu);
            for (int64_t i = start; i < end; ++i) payload[i] = 0;
            continue;
        }
        float scale = maximum > 0.0f ? maximum / 127.0f : 1.0f;
        scales[b] = scale;
        for (int64_t i = start; i < end; ++i)
            payload[i] = code_from_quotient(source[i] / scale);
    }
    return ORACLE_OK;
}

/*
 * Tensor-wide gradient publication (the pure-BFP8 reducer's local step):
 * finite check, scale, payload, decode written back over the fp32 gradient,
 * optional sum of squares of the decoded values.
 * NNtrain.Cuda/native/tensor_kernels.cu:988-1073,1114-1146.
 * A non-finite input sets *finite_status = 1, forces scale = 1 and leaves
 * payload and gradient untouched (:1015-1018,1027,1038); the sum of squares
 * still runs over whatever the payload buffer holds (:1141-1144).
 * `block` = 0 gives the reference's tensor-wide behaviour; a positive block
 * applies the same publication per block (the N-rank extension).
 */
int oracle_bfp8_gradient_publish(float* gradient, int64_t length, int64_t block,
                                 int8_t* payload, float* scales,
                                 int* finite_status, double* squared_sum) {
    if (!gradient || !payload || !scales || !finite_status || length <= 0)
        return ORACLE_ERR_ARGUMENT;
    const int64_t eb = effective_block(length, block);
    const int64_t count = (length + eb - 1) / eb;
    int non_finite = *finite_status != 0;
    for (int64_t i = 0; i < length && !non_finite; ++i)
        if (!isfinite(gradient[i])) non_finite = 1;
    if (non_finite) {
        *finite_status = 1;
        for (int64_t b = 0; b < count; ++b) scales[b] = 1.0f;
    } else {
        int rc = oracle_bfp8_encode(gradient, length, block, payload, scales, 0);
        if (rc != ORACLE_OK) return rc;
        oracle_bfp8_decode(payload, scales, length, block, gradient, 0);
    }
    if (squared_sum) {
        double total = 0.0;
        #pragma omp parallel for reduction(+:total) schedule(static)
        for (int64_t i = 0; i < length; ++i) {
            float s = scales[i / eb];
            if (isfinite(s) && s > 0.0f) {
                double d = (double)((float)payload[i] * s);
                total += d * d;
            }
        }
        *squared_sum += total;
    }
    return ORACLE_OK;
}

/*
 * BF16 encode.  rule 0: the C# codec, NNtrain.Core/Tensors/TensorStorage.cs:
 * 758-767 (NaN keeps its top bits and gets the quiet bit; otherwise
 * bits + 0x7FFF + lsb, take the top half).  rule 1: CUDA's
 * __float2bfloat16_rn as used by the bucket pack kernel
 * (NNtrain.Cuda/native/gradient_collectives.cu:11-22), which differs only in
 * mapping every NaN to 0x7FFF.
 */
uint16_t oracle_bf16_encode_one(float value, int rule) {
    uint32_t bits = f32_bits(value);
    uint32_t absolute = bits & 0x7FFFFFFFu;
    if (absolute > 0x7F800000u)
        return rule == 0 ? (uint16_t)((bits >> 16) | 0x0040u) : (uint16_t)0x7FFFu;
    uint32_t rounded = bits + 0x7FFFu + ((bits >> 16) & 1u);
    return (uint16_t)(rounded >> 16);
}

int oracle_bf16_encode(const float* source, int64_t length, uint16_t* destination, int rule) {
    if (!source || !destination || length <= 0) return ORACLE_ERR_ARGUMENT;
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < length; ++i)
        destination[i] = oracle_bf16_encode_one(source[i], rule);
    return ORACLE_OK;
}

/* BF16 decode: bits << 16.  TensorStorage.cs:769-770. */
int oracle_bf16_decode(const uint16_t* source, int64_t length, float* destination) {
    if (!source || !destination || length <= 0) return ORACLE_ERR_ARGUMENT;
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < length; ++i)
        destination[i] = bits_f32((uint32_t)source[i] << 16);
    return ORACLE_OK;
}

/*
 * BF16 transport sum over N ranks, fp32 accumulate in ascending rank order:
 * reduced = fl(f32(a) + f32(b)) (+ ...).
 * NNtrain.Cuda/native/gradient_collectives.cu:62-90;
 * NNtrain.Core.Tests/CudaMix8GradientTransportTests.cs:83-88.
 * bf16_out (optional): the arena mode's authoritative re-encoded result
 * (NNtrain.Core/Training/CudaBFloat16GradientAllReduce.cs:1413-1459).
 * squared_sum (optional) accumulates (double)v*v of the fp32 sum, or of the
 * bf16-rounded value when square_of_bf16 != 0.
 */
int oracle_bf16_reduce(const uint16_t* const* inputs, int ranks, int64_t length,
                       float reduction_scale, float* reduced, uint16_t* bf16_out,
                       double* squared_sum, int square_of_bf16) {
    if (!inputs || ranks < 1 || length <= 0 || (!reduced && !bf16_out))
        return ORACLE_ERR_ARGUMENT;
    double total = 0.0;
    #pragma omp parallel for reduction(+:total) schedule(static)
    for (int64_t i = 0; i < length; ++i) {
        float sum = bits_f32((uint32_t)inputs[0][i] << 16);
        for (int r = 1; r < ranks; ++r)
            sum = sum + bits_f32((uint32_t)inputs[r][i] << 16);
        sum = reduction_scale * sum;
        if (reduced) reduced[i] = sum;
        float squared_of = sum;
        if (bf16_out) {
            uint16_t e = oracle_bf16_encode_one(sum, 1);
            bf16_out[i] = e;
            if (square_of_bf16) squared_of = bits_f32((uint32_t)e << 16);
        }
        total += (double)squared_of * (double)squared_of;
    }
    if (squared_sum) *squared_sum += total;
    return ORACLE_OK;
}

/* Sum of squares in binary64.  NNtrain.Core/Torch/nn.cs:62-67;
 * NNtrain.Cuda/native/tensor_kernels.cu:968-986. */
double oracle_squared_sum_f32(const float* values, int64_t length) {
    double total = 0.0;
    #pragma omp parallel for reduction(+:total) schedule(static)
    for (int64_t i = 0; i < length; ++i) total += (double)values[i] * (double)values[i];
    return total;
}

double oracle_squared_sum_bf16(const uint16_t* values, int64_t length) {
    double total = 0.0;
    #pragma omp parallel for reduction(+:total) schedule(static)
    for (int64_t i = 0; i < length; ++i) {
        double v = (double)bits_f32((uint32_t)values[i] << 16);
        total += v * v;
    }
    return total;
}

/* Sum of squares of the decoded BFP8 values, skipping blocks whose scale is
 * invalid.  NNtrain.Cuda/native/tensor_kernels.cu:1047-1073. */
double oracle_squared_sum_bfp8(const int8_t* payload, const float* scales,
                               int64_t length, int64_t block) {
    const int64_t eb = effective_block(length, block);
    double total = 0.0;
    #pragma omp parallel for reduction(+:total) schedule(static)
    for (int64_t i = 0; i < length; ++i) {
        float s = scales[i / eb];
        if (isfinite(s) && s > 0.0f) {
            double d = (double)((float)payload[i] * s);
            total += d * d;
        }
    }
    return total;
}

/*
 * Global clip coefficient.  NNtrain.Core/Torch/nn.cs:69-81:
 *   norm = (float)sqrt(sum_sq); clip iff norm > max_norm;
 *   coefficient = max_norm / (norm + 1e-6f)   (binary32).
 * Returns the pre-clip norm; *coefficient = 1 when no clip applies.
 */
float oracle_clip_coefficient(double squared_sum, float max_norm, float* coefficient) {
    float norm = (float)sqrt(squared_sum);
    float c = 1.0f;
    if (norm > max_norm) c = max_norm / (norm + 1e-6f);
    if (coefficient) *coefficient = c;
    return norm;
}

/* Clip applied to fp32 values: g *= c.  nn.cs:72-78; tensor_kernels.cu:910-914. */
void oracle_scale_f32(float* values, int64_t length, float multiplier) {
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < length; ++i) values[i] = values[i] * multiplier;
}

/* Clip applied to bf16 values: g = bf16_rn(f32(g) * c).
 * NNtrain.Cuda/native/pure_bfloat16_gradients.cu:337-348. */
void oracle_scale_bf16(uint16_t* values, int64_t length, float multiplier) {
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < length; ++i)
        values[i] = oracle_bf16_encode_one(bits_f32((uint32_t)values[i] << 16) * multiplier, 1);
}

/* Clip applied to BFP8: scale-only, payload untouched;
 * scale = fmaxf(scale * c, FLT_MIN).  tensor_kernels.cu:1075-1082. */
void oracle_scale_bfp8_scales(float* scales, int64_t count, float multiplier) {
    for (int64_t i = 0; i < count; ++i) {
        float v = scales[i] * multiplier;
        scales[i] = (v != v) ? FLT_MIN : (v > FLT_MIN ? v : FLT_MIN);
    }
}

/* ------------------------------------------------------------------------
 * Seeded synthetic gradients (not from the reference: the workloads'
 * inputs).  Counter-based so any slice can be regenerated independently:
 *   u = splitmix64(seed ^ (replica << 48) ^ index); two 24-bit uniforms ->
 *   Box-Muller in binary64 -> * sigma -> binary32.
 * ---------------------------------------------------------------------- */
static inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

static inline double unit_normal(uint64_t seed, uint64_t replica, uint64_t index) {
    uint64_t u = splitmix64(seed ^ (replica << 48) ^ index);
    double u1 = ((double)((u >> 40) & 0xFFFFFFull) + 1.0) / 16777217.0;   /* (0,1) */
    double u2 = (double)((u >> 16) & 0xFFFFFFull) / 16777216.0;           /* [0,1) */
    return sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2);
}

/*
 * Gradient-like data: N(0, sigma) with sigma log-uniform in
 * [sigma_lo, sigma_hi] per `slice` elements; a fraction `outlier_fraction`
 * of 32-value blocks scaled x100; a fraction `zero_fraction` of 32-value
 * blocks all zero; `subnormals` elements overwritten with values in
 * [1e-40, 1e-39] at positions inside blocks whose maximum is normal.
 * `offset` is the index of destination[0] within the replica's full
 * gradient of `total_length` elements, so slices of one logical arena can be generated independently.
 */
void oracle_generate_gradient(float* destination, int64_t length, int64_t offset,
                              int64_t total_length, uint64_t seed, uint64_t replica, int64_t slice,
                              double sigma_lo, double sigma_hi,
                              double outlier_fraction, double zero_fraction,
                              int subnormals) {
    const double log_lo = log10(sigma_lo), log_hi = log10(sigma_hi);
    #pragma omp parallel for schedule(static)
    for (int64_t k = 0; k < length; ++k) {
        const uint64_t index = (uint64_t)(offset + k);
        const uint64_t slice_id = slice > 0 ? index / (uint64_t)slice : 0;
        /* sigma depends on the slice only (same for every replica) */
        uint64_t hs = splitmix64(seed ^ 0x5151515151515151ull ^ (slice_id * 0x100000001B3ull));
        double us = (double)(hs >> 11) / 9007199254740992.0;
        double sigma = pow(10.0, log_lo + (log_hi - log_lo) * us);
        /* block class depends on replica and 32-block */
        const uint64_t block_id = index >> 5;
        uint64_t hb = splitmix64(seed ^ 0xA5A5A5A5A5A5A5A5ull ^ (replica << 48) ^ (block_id * 0x9E3779B1ull));
        double ub = (double)(hb >> 11) / 9007199254740992.0;
        double v = unit_normal(seed, replica, index) * sigma;
        if (ub < zero_fraction) v = 0.0;
        else if (ub < zero_fraction + outlier_fraction) v *= 100.0;
        destination[k] = (float)v;
    }
    /* a few subnormal values, at fixed pseudo-random positions of the replica */
    for (int s = 0; s < subnormals; ++s) {
        uint64_t h = splitmix64(seed ^ 0x0123456789ABCDEFull ^ (replica << 48) ^ (uint64_t)s);
        int64_t pos = (int64_t)(h % (uint64_t)(total_length > 0 ? total_length : 1));
        if (pos < offset || pos >= offset + length) continue;
        float tiny = (float)(1e-40 + 9e-40 * (double)((h >> 20) & 0xFFFF) / 65536.0);
        destination[pos - offset] = ((h >> 63) ? -tiny : tiny);
    }
}
