// Loader kernels: re-lay the .cimage split-block payload into the device
// layout (common.cuh), its inverse, the bit-exact dequantiser, the embedding
// row gather and the on-device synthetic weight generator.
#include "common.cuh"

namespace prism {

// One thread per 16-byte unit (hb, chunk, lane) of the device index array.
// Source: reference payload of a [src_m][src_k] tensor -- palettes first
// (src_m * 2^bits * 2 bytes), then row-major packed index rows
// (src/lut/compiler.rs:50-61).  A shard starts at (row0, col0).
__global__ void relay_idx_kernel(const uint8_t *__restrict__ payload, uint32_t src_m,
                                 uint32_t src_row_bytes, uint32_t n_ent, uint32_t row0,
                                 uint32_t byte0, uint32_t m, uint32_t row_bytes, uint32_t n_chunks,
                                 uint32_t n_hb, uint8_t *__restrict__ idx) {
    size_t unit = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)n_hb * n_chunks * 32;
    if (unit >= total) return;
    uint32_t lane = (uint32_t)(unit & 31);
    size_t hc = unit >> 5;
    uint32_t chunk = (uint32_t)(hc % n_chunks);
    uint32_t hb = (uint32_t)(hc / n_chunks);
    uint32_t row = hb * 32 + lane;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < m) {
        const uint8_t *src = payload + (size_t)src_m * n_ent * 2 +
                             (size_t)(row0 + row) * src_row_bytes + byte0 + (size_t)chunk * 16;
        uint32_t valid = row_bytes - chunk * 16;
        if (valid > 16) valid = 16;
        if (valid == 16 && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
            v = *reinterpret_cast<const uint4 *>(src);
        } else {
            __align__(16) uint8_t b[16];
#pragma unroll
            for (int i = 0; i < 16; i++) b[i] = (uint32_t)i < valid ? src[i] : (uint8_t)0;
            const uint32_t *w = reinterpret_cast<const uint32_t *>(b);
            v = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
    *reinterpret_cast<uint4 *>(idx + unit * 16) = v;
}

__global__ void relay_pal_kernel(const uint8_t *__restrict__ payload, uint32_t n_ent, uint32_t row0,
                                 uint32_t m, uint32_t m_pad, uint16_t *__restrict__ pal) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)m_pad * n_ent;
    if (i >= total) return;
    uint32_t row = (uint32_t)(i / n_ent);
    uint16_t v = 0;
    if (row < m) {
        const uint8_t *s = payload + ((size_t)(row0 + row) * n_ent + (i % n_ent)) * 2;
        v = (uint16_t)(s[0] | ((uint16_t)s[1] << 8));
    }
    pal[i] = v;
}

int launch_relay(prism_cuda_ctx *ctx, const uint8_t *payload_dev, uint32_t src_m, uint32_t src_k,
                 uint32_t row0, uint32_t col0, LutTensor &t) {
    uint32_t src_row_bytes = src_k * t.bits / 8;
    uint32_t byte0 = col0 * t.bits / 8;
    size_t units = (size_t)t.n_hb * t.n_chunks * 32;
    if (units) {
        relay_idx_kernel<<<(unsigned)((units + 255) / 256), 256, 0, ctx->stream>>>(
            payload_dev, src_m, src_row_bytes, t.n_ent(), row0, byte0, t.m, t.row_bytes, t.n_chunks,
            t.n_hb, t.idx);
        PRISM_TRY(after_launch(ctx, "relay_idx_kernel"));
    }
    size_t pe = (size_t)t.m_pad * t.n_ent();
    relay_pal_kernel<<<(unsigned)((pe + 255) / 256), 256, 0, ctx->stream>>>(payload_dev, t.n_ent(), row0,
                                                                           t.m, t.m_pad, t.pal);
    return after_launch(ctx, "relay_pal_kernel");
}

// Inverse: device layout -> reference payload of the [m][k] tensor.
__global__ void unrelay_kernel(const uint8_t *__restrict__ idx, const uint16_t *__restrict__ pal,
                               uint32_t m, uint32_t row_bytes, uint32_t n_chunks, uint32_t n_ent,
                               uint8_t *__restrict__ payload) {
    size_t unit = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)((m + 31) / 32) * n_chunks * 32;
    if (unit >= total) return;
    uint32_t lane = (uint32_t)(unit & 31);
    size_t hc = unit >> 5;
    uint32_t chunk = (uint32_t)(hc % n_chunks);
    uint32_t hb = (uint32_t)(hc / n_chunks);
    uint32_t row = hb * 32 + lane;
    if (row >= m) return;
    uint8_t *dst = payload + (size_t)m * n_ent * 2 + (size_t)row * row_bytes + (size_t)chunk * 16;
    const uint8_t *src = idx + unit * 16;
    uint32_t valid = row_bytes - chunk * 16;
    if (valid > 16) valid = 16;
    for (uint32_t i = 0; i < valid; i++) dst[i] = src[i];
    if (chunk == 0) {
        for (uint32_t e = 0; e < n_ent; e++) {
            uint16_t v = pal[(size_t)row * n_ent + e];
            payload[((size_t)row * n_ent + e) * 2] = (uint8_t)(v & 0xFF);
            payload[((size_t)row * n_ent + e) * 2 + 1] = (uint8_t)(v >> 8);
        }
    }
}

int launch_unrelay(prism_cuda_ctx *ctx, const LutTensor &t, uint8_t *payload_dev) {
    size_t units = (size_t)((t.m + 31) / 32) * t.n_chunks * 32;
    unrelay_kernel<<<(unsigned)((units + 255) / 256), 256, 0, ctx->stream>>>(
        t.idx, t.pal, t.m, t.row_bytes, t.n_chunks, t.n_ent(), payload_dev);
    return after_launch(ctx, "unrelay_kernel");
}

// W[r][k] = palette[r][index(r,k)] as the stored bit pattern
// (PrismEngine::embed, src/lut/engine_impl.rs:1407-1446).  One thread per
// 16-byte unit; writes 32 (4-bit) or 64 (2-bit) fp16 values.
template <int BITS>
__global__ void dequant_kernel(const uint8_t *__restrict__ idx, const uint16_t *__restrict__ pal,
                               uint32_t m, uint32_t k, uint32_t n_chunks, uint32_t n_hb,
                               uint16_t *__restrict__ out) {
    constexpr uint32_t NE = 1u << BITS, PER_CHUNK = 128 / BITS, MASK = NE - 1;
    size_t unit = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)n_hb * n_chunks * 32;
    if (unit >= total) return;
    uint32_t lane = (uint32_t)(unit & 31);
    size_t hc = unit >> 5;
    uint32_t chunk = (uint32_t)(hc % n_chunks);
    uint32_t hb = (uint32_t)(hc / n_chunks);
    uint32_t row = hb * 32 + lane;
    if (row >= m) return;
    uint4 v = *reinterpret_cast<const uint4 *>(idx + unit * 16);
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
    const uint16_t *p = pal + (size_t)row * NE;
    uint32_t k0 = chunk * PER_CHUNK;
#pragma unroll
    for (uint32_t i = 0; i < PER_CHUNK; i++) {
        uint32_t kk = k0 + i;
        if (kk < k) {
            uint32_t bit = i * BITS;
            out[(size_t)row * k + kk] = p[(w[bit >> 5] >> (bit & 31)) & MASK];
        }
    }
}

int launch_dequant(prism_cuda_ctx *ctx, const LutTensor &t, uint16_t *out_dev) {
    size_t units = (size_t)t.n_hb * t.n_chunks * 32;
    unsigned grid = (unsigned)((units + 127) / 128);
    if (t.bits == 4)
        dequant_kernel<4><<<grid, 128, 0, ctx->stream>>>(t.idx, t.pal, t.m, t.k, t.n_chunks, t.n_hb, out_dev);
    else
        dequant_kernel<2><<<grid, 128, 0, ctx->stream>>>(t.idx, t.pal, t.m, t.k, t.n_chunks, t.n_hb, out_dev);
    return after_launch(ctx, "dequant_kernel");
}

// Embedding row gather for `batch` tokens: out[b][:] = dequantised row
// tokens[b], zeros when the id is out of range (engine_impl.rs:1423-1425).
// out2 (optional) receives the same values (the residual copy `hr = h.clone()`,
// engine_impl.rs:1083).
template <int BITS>
__global__ void embed_kernel(const uint8_t *__restrict__ idx, const uint16_t *__restrict__ pal,
                             uint32_t m, uint32_t k, uint32_t n_chunks,
                             const uint32_t *__restrict__ tokens, uint16_t *__restrict__ out,
                             uint16_t *__restrict__ out2) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr uint32_t NE = 1u << BITS, PER_CHUNK = 128 / BITS, MASK = NE - 1;
    uint32_t b = blockIdx.y;
    uint32_t tok = tokens[b];
    for (uint32_t chunk = blockIdx.x * blockDim.x + threadIdx.x; chunk < n_chunks;
         chunk += gridDim.x * blockDim.x) {
        uint32_t k0 = chunk * PER_CHUNK;
        if (tok >= m) {
            for (uint32_t i = 0; i < PER_CHUNK && k0 + i < k; i++) {
                out[(size_t)b * k + k0 + i] = 0;
                if (out2) out2[(size_t)b * k + k0 + i] = 0;
            }
            continue;
        }
        uint32_t hb = tok >> 5, lane = tok & 31;
        uint4 v = *reinterpret_cast<const uint4 *>(idx + lut_idx_offset(n_chunks, hb, chunk, lane));
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
        const uint16_t *p = pal + (size_t)tok * NE;
#pragma unroll
        for (uint32_t i = 0; i < PER_CHUNK; i++) {
            uint32_t kk = k0 + i;
            if (kk < k) {
                uint32_t bit = i * BITS;
                uint16_t e = p[(w[bit >> 5] >> (bit & 31)) & MASK];
                out[(size_t)b * k + kk] = e;
                if (out2) out2[(size_t)b * k + kk] = e;
            }
        }
    }
}

int launch_embed(prism_cuda_ctx *ctx, const LutTensor &t, const uint32_t *tokens_dev, uint32_t batch,
                 uint16_t *out_dev, uint16_t *out2_dev) {
    dim3 grid((t.n_chunks + 63) / 64, batch);
    if (t.bits == 4)
        launch_pdl(ctx, "embed_kernel", embed_kernel<4>, grid, 64, 0, t.idx, t.pal, t.m, t.k, t.n_chunks, tokens_dev, out_dev, out2_dev);
    else
        launch_pdl(ctx, "embed_kernel", embed_kernel<2>, grid, 64, 0, t.idx, t.pal, t.m, t.k, t.n_chunks, tokens_dev, out_dev, out2_dev);
    return after_launch(ctx, "embed_kernel");
}

// ---- synthetic weights, generated in place in the device layout -----------

__device__ inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// Index bytes: uniform, a pure function of (seed, row, byte position in the row).
__global__ void synth_idx_kernel(uint64_t seed, uint32_t m, uint32_t row_bytes, uint32_t n_chunks,
                                 uint32_t n_hb, uint32_t row0, uint32_t chunk0, uint8_t *__restrict__ idx) {
    size_t unit = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t total = (size_t)n_hb * n_chunks * 32;
    if (unit >= total) return;
    uint32_t lane = (uint32_t)(unit & 31);
    size_t hc = unit >> 5;
    uint32_t chunk = (uint32_t)(hc % n_chunks);
    uint32_t hb = (uint32_t)(hc / n_chunks);
    uint32_t row = hb * 32 + lane;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < m) {
        uint64_t base = seed ^ (((uint64_t)(row0 + row) << 32) | (chunk0 + chunk));
        uint64_t a = splitmix64(base), b = splitmix64(base ^ 0xD1B54A32D192ED03ull);
        v = make_uint4((uint32_t)a, (uint32_t)(a >> 32), (uint32_t)b, (uint32_t)(b >> 32));
        uint32_t valid = row_bytes - chunk * 16;
        if (valid < 16) {
            uint8_t *pb = reinterpret_cast<uint8_t *>(&v);
            for (uint32_t i = valid; i < 16; i++) pb[i] = 0;
        }
    }
    *reinterpret_cast<uint4 *>(idx + unit * 16) = v;
}

// Palette: 2^bits values ~ N(0, sigma) (Box-Muller over splitmix64), sorted
// ascending, rounded to fp16.  One thread per row.
__global__ void synth_pal_kernel(uint64_t seed, uint32_t m, uint32_t m_pad, uint32_t n_ent, float sigma,
                                 uint32_t row0, uint16_t *__restrict__ pal) {
    uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= m_pad) return;
    float v[16];
    for (uint32_t e = 0; e < n_ent; e++) {
        uint64_t h = splitmix64(seed ^ 0xA5A5A5A5ull ^ (((uint64_t)(row0 + row) << 8) | e));
        float u1 = ((uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777217.0f);
        float u2 = (uint32_t)((h >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);
        v[e] = sigma * sqrtf(-2.0f * logf(u1)) * cosf(6.2831853071795865f * u2);
    }
    for (uint32_t i = 1; i < n_ent; i++) {
        float x = v[i];
        uint32_t j = i;
        while (j > 0 && v[j - 1] > x) {
            v[j] = v[j - 1];
            j--;
        }
        v[j] = x;
    }
    for (uint32_t e = 0; e < n_ent; e++)
        pal[(size_t)row * n_ent + e] = row < m ? __half_as_ushort(__float2half_rn(v[e])) : (uint16_t)0;
}

// (row0, col0): position of this tensor inside the full tensor it is a shard of, so a
// tensor-parallel rank generates exactly its slice of the single-GPU weights.
int launch_synth(prism_cuda_ctx *ctx, LutTensor &t, uint64_t seed, float sigma, uint32_t row0, uint32_t col0) {
    const uint32_t chunk0 = col0 * t.bits / 128;
    size_t units = (size_t)t.n_hb * t.n_chunks * 32;
    synth_idx_kernel<<<(unsigned)((units + 255) / 256), 256, 0, ctx->stream>>>(seed, t.m, t.row_bytes,
                                                                              t.n_chunks, t.n_hb, row0, chunk0, t.idx);
    PRISM_TRY(after_launch(ctx, "synth_idx_kernel"));
    synth_pal_kernel<<<(t.m_pad + 127) / 128, 128, 0, ctx->stream>>>(seed, t.m, t.m_pad, t.n_ent(), sigma, row0, t.pal);
    return after_launch(ctx, "synth_pal_kernel");
}

}  // namespace prism
