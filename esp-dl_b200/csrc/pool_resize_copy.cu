// Pooling, nearest-neighbour resize and strided copy (Concat / Split / Transpose / Slice).
// All bandwidth bound; threads run along the channel axis so every warp access is contiguous.
//   MaxPool            esp-dl/dl/base/dl_base_max_pool2d.cpp:9-27 (in-bounds taps only)
//   (Global)AveragePool esp-dl/dl/base/dl_base_avg_pool2d.cpp:10-55 (int sum, fp32 scale, area = kh*kw)
//   Resize nearest     esp-dl/dl/base/dl_base_resize.cpp:7-35,239-279
//   Concat             esp-dl/dl/module/include/dl_module_concat.hpp:87-107
#include "common.cuh"

namespace espdl {

struct PoolParams {
    const void *in;
    void *out;
    int op, is16, n, ih, iw, c, oh, ow, kh, kw, sh, sw, pt, pl;
    float scale;
    long long total;
};

__global__ void __launch_bounds__(256) pool_kernel(PoolParams p)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < p.total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % p.c);
        const long long pix = i / p.c;
        const int ox = (int)(pix % p.ow);
        const int oy = (int)((pix / p.ow) % p.oh);
        const int n = (int)(pix / ((long long)p.ow * p.oh));
        long long sum = 0;
        int mx = INT32_MIN;
        for (int ky = 0; ky < p.kh; ky++) {
            const int iy = oy * p.sh + ky - p.pt;
            if (iy < 0 || iy >= p.ih)
                continue;
            for (int kx = 0; kx < p.kw; kx++) {
                const int ix = ox * p.sw + kx - p.pl;
                if (ix < 0 || ix >= p.iw)
                    continue;
                const long long ii = (((long long)n * p.ih + iy) * p.iw + ix) * p.c + c;
                const int v = p.is16 ? (int)((const int16_t *)p.in)[ii] : (int)((const int8_t *)p.in)[ii];
                sum += v;
                mx = max(mx, v);
            }
        }
        int r;
        if (p.op == ESPDL_POOL_MAX) {
            r = mx;
        } else {
            // int8: the reference accumulates in int32, int16: in int64; both convert the sum to fp32
            const float f = p.is16 ? __ll2float_rn(sum) : __int2float_rn((int)sum);
            r = fround_half_up(__fmul_rn(f, p.scale));
        }
        if (p.is16)
            ((int16_t *)p.out)[i] = (int16_t)sat16(r);
        else
            ((int8_t *)p.out)[i] = (int8_t)sat8(r);
    }
}

// Max pool, int8, C % 16 == 0: 16 channels per thread, 128-bit loads and stores, per-byte signed maximum over the
// in-bounds taps (padding is excluded, as in pool_kernel).
__global__ void __launch_bounds__(256) maxpool_s8_vec16_kernel(PoolParams p)
{
    const int chunks = p.c >> 4;
    const long long total = (long long)p.n * p.oh * p.ow * chunks;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int ch = (int)(i % chunks) * 16;
        const long long pix = i / chunks;
        const int ox = (int)(pix % p.ow);
        const int oy = (int)((pix / p.ow) % p.oh);
        const int n = (int)(pix / ((long long)p.ow * p.oh));
        uint4 m = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u); // -128 in every byte
        for (int ky = 0; ky < p.kh; ky++) {
            const int iy = oy * p.sh + ky - p.pt;
            if (iy < 0 || iy >= p.ih)
                continue;
            for (int kx = 0; kx < p.kw; kx++) {
                const int ix = ox * p.sw + kx - p.pl;
                if (ix < 0 || ix >= p.iw)
                    continue;
                const uint4 v = __ldg((const uint4 *)((const int8_t *)p.in + (((long long)n * p.ih + iy) * p.iw + ix) * p.c + ch));
                m.x = __vmaxs4(m.x, v.x), m.y = __vmaxs4(m.y, v.y), m.z = __vmaxs4(m.z, v.z), m.w = __vmaxs4(m.w, v.w);
            }
        }
        *(uint4 *)((int8_t *)p.out + pix * p.c + ch) = m;
    }
}

// Stride-1 K x K max pool (the detector's 5x5 pools), int8, C % 16 == 0: a thread owns 16 channels of one output COLUMN and
// walks down the image.  Per input row it takes the maximum over the K columns of the window once (K loads), keeps
// the last K of these row maxima in registers and emits one output per row as their maximum: K loads and 2(K - 1)
// maxima per output instead of K*K of each.  Bytes are compared as the high bytes of 16-bit lanes (even and odd
// bytes of a word apart), where the packed 16-bit maximum is one instruction.  The row loop is unrolled by K so that
// the ring of row maxima is indexed statically.  Taps outside the image are left out, as in pool_kernel.
struct Lanes16 {
    uint32_t e[4], o[4]; // even / odd bytes of four words, each in the high byte of a 16-bit lane
};

__device__ __forceinline__ void split_bytes(const uint4 v, Lanes16 &l)
{
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) l.e[i] = (w[i] << 8) & 0xff00ff00u, l.o[i] = w[i] & 0xff00ff00u;
}

// max.s16x2 is one instruction on this architecture (the __vmaxs2 intrinsic expands to several)
__device__ __forceinline__ uint32_t max_s16x2(uint32_t a, uint32_t b)
{
    uint32_t r;
    asm("max.s16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

__device__ __forceinline__ void max_lanes(Lanes16 &a, const Lanes16 &b)
{
#pragma unroll
    for (int i = 0; i < 4; i++) a.e[i] = max_s16x2(a.e[i], b.e[i]), a.o[i] = max_s16x2(a.o[i], b.o[i]);
}

template <int K>
__global__ void __launch_bounds__(256) maxpool_s8_walk_kernel(PoolParams p, int segments)
{
    const int chunks = p.c >> 4;
    const int seg_rows = (p.oh + segments - 1) / segments; // a column is cut into `segments` runs of output rows when there are few columns
    const long long total = (long long)p.n * segments * p.ow * chunks;
    for (long long item = blockIdx.x * (long long)blockDim.x + threadIdx.x; item < total; item += (long long)gridDim.x * blockDim.x) {
        const int ch = (int)(item % chunks) * 16;
        const int ox = (int)((item / chunks) % p.ow);
        const int seg = (int)((item / ((long long)chunks * p.ow)) % segments);
        const long long n = item / ((long long)chunks * p.ow * segments);
        const int oy0 = seg * seg_rows, oy1 = min(p.oh, oy0 + seg_rows);
        const int8_t *in = (const int8_t *)p.in + n * p.ih * (long long)p.iw * p.c + ch;
        int8_t *out = (int8_t *)p.out + (n * p.oh * (long long)p.ow + ox) * p.c + ch;
        // taps outside the image count as -128, the identity of the maximum (every window holds at least one real tap)
        Lanes16 ring[K];
#pragma unroll
        for (int j = 0; j < K; j++)
#pragma unroll
            for (int i = 0; i < 4; i++) ring[j].e[i] = ring[j].o[i] = 0x80008000u;
        const int last_iy = oy1 - 1 + K - 1 - p.pt; // the input row (possibly below the image) that completes the run's last output row
        const int first_iy = max(oy0 - p.pt, 0);
#pragma unroll 1
        for (int base = first_iy / K * K; base <= last_iy; base += K) {
#pragma unroll
            for (int j = 0; j < K; j++) {
                const int iy = base + j;
                const bool row_in = iy >= first_iy && iy < p.ih;
                const int8_t *row = in + (long long)min(iy, p.ih - 1) * p.iw * p.c;
                uint4 v[K]; // all K loads of the row are issued before the first is used
#pragma unroll
                for (int kx = 0; kx < K; kx++) {
                    const int x = ox - p.pl + kx;
                    v[kx] = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
                    if (row_in && x >= 0 && x < p.iw)
                        v[kx] = __ldg((const uint4 *)(row + (long long)x * p.c));
                }
                split_bytes(v[0], ring[j]);
#pragma unroll
                for (int kx = 1; kx < K; kx++) {
                    Lanes16 t;
                    split_bytes(v[kx], t);
                    max_lanes(ring[j], t);
                }
                const int oy = iy - (K - 1) + p.pt; // its window is input rows iy - K + 1 .. iy
                if (oy >= oy0 && oy < oy1) {
                    Lanes16 m = ring[0];
#pragma unroll
                    for (int d = 1; d < K; d++) max_lanes(m, ring[d]);
                    uint4 o;
                    o.x = (m.e[0] >> 8) | m.o[0], o.y = (m.e[1] >> 8) | m.o[1], o.z = (m.e[2] >> 8) | m.o[2], o.w = (m.e[3] >> 8) | m.o[3];
                    *(uint4 *)(out + (long long)oy * p.ow * p.c) = o;
                }
            }
        }
    }
}

// Global average pool, int8, C % 4 == 0: a thread owns four channels (one word of each pixel) of one image and sums
// the whole plane; lanes are consecutive words, so every load of a warp is one contiguous run.  The four byte sums
// come from dp4a against one-hot byte selectors.  Same arithmetic as pool_kernel (int32 sum, one fp32 multiply).
__global__ void __launch_bounds__(256) gap_s8_kernel(PoolParams p)
{
    const int quads = p.c >> 2;
    const long long item = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (item >= (long long)p.n * quads)
        return;
    const int q = (int)(item % quads);
    const long long n = item / quads;
    const int pixels = p.ih * p.iw;
    const uint32_t *src = (const uint32_t *)((const int8_t *)p.in + n * (long long)pixels * p.c) + q;
    int s0 = 0, s1 = 0, s2 = 0, s3 = 0;
#pragma unroll 7
    for (int i = 0; i < pixels; i++) {
        const int w = (int)__ldg(src + (long long)i * quads);
        s0 = __dp4a(w, 0x00000001, s0);
        s1 = __dp4a(w, 0x00000100, s1);
        s2 = __dp4a(w, 0x00010000, s2);
        s3 = __dp4a(w, 0x01000000, s3);
    }
    const int r0 = sat8(fround_half_up(__fmul_rn(__int2float_rn(s0), p.scale)));
    const int r1 = sat8(fround_half_up(__fmul_rn(__int2float_rn(s1), p.scale)));
    const int r2 = sat8(fround_half_up(__fmul_rn(__int2float_rn(s2), p.scale)));
    const int r3 = sat8(fround_half_up(__fmul_rn(__int2float_rn(s3), p.scale)));
    ((uint32_t *)p.out)[item] = (uint32_t)(r0 & 0xff) | ((uint32_t)(r1 & 0xff) << 8) | ((uint32_t)(r2 & 0xff) << 16) | ((uint32_t)(r3 & 0xff) << 24);
}

struct ResizeParams {
    const int8_t *in;
    int8_t *out;
    int n, ih, iw, c, oh, ow, ops, two;
    float sh_inv, sw_inv, oscale, odiv;
    long long total;
};

__global__ void __launch_bounds__(256) resize_nearest_kernel(ResizeParams p)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < p.total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % p.c);
        const long long pix = i / p.c;
        const int x = (int)(pix % p.ow);
        const int y = (int)((pix / p.ow) % p.oh);
        const int n = (int)(pix / ((long long)p.ow * p.oh));
        int iy = p.two ? y / 2 : (int)__fmul_rn((float)y, p.sh_inv);
        int ix = p.two ? x / 2 : (int)__fmul_rn((float)x, p.sw_inv);
        iy = min(iy, p.ih - 1);
        ix = min(ix, p.iw - 1);
        const int v = p.in[(((long long)n * p.ih + iy) * p.iw + ix) * p.c + c];
        // (float)x * scale / (1 << shift), then round; the reference stores the result with a plain cast
        const float f = __fdiv_rn(__fmul_rn((float)v, p.oscale), p.odiv);
        p.out[pix * p.ops + c] = (int8_t)fround_half_up(f);
    }
}

// Nearest resize with equal input and output exponents is a pure gather ((float)q * 1 / 1 rounds back to q): 16
// channels per thread, 128-bit loads and stores, a warp moves contiguous runs of both tensors.
__global__ void __launch_bounds__(256) resize_nearest_vec16_kernel(ResizeParams p)
{
    const int chunks = p.c >> 4;
    const long long total = (long long)p.n * p.oh * p.ow * chunks;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int ch = (int)(i % chunks) * 16;
        const long long pix = i / chunks;
        const int x = (int)(pix % p.ow);
        const int y = (int)((pix / p.ow) % p.oh);
        const int n = (int)(pix / ((long long)p.ow * p.oh));
        int iy = p.two ? y / 2 : (int)__fmul_rn((float)y, p.sh_inv);
        int ix = p.two ? x / 2 : (int)__fmul_rn((float)x, p.sw_inv);
        iy = min(iy, p.ih - 1);
        ix = min(ix, p.iw - 1);
        const uint4 v = __ldg((const uint4 *)(p.in + (((long long)n * p.ih + iy) * p.iw + ix) * p.c + ch));
        *(uint4 *)(p.out + pix * p.ops + ch) = v;
    }
}

struct CopyParams {
    const char *src;
    char *dst;
    int es;
    int shape[6];
    long long ss[6], ds[6];
    long long total;
};

template <typename T>
__global__ void __launch_bounds__(256) copy_kernel(CopyParams p)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < p.total; i += (long long)gridDim.x * blockDim.x) {
        long long r = i, si = 0, di = 0;
#pragma unroll
        for (int k = 5; k >= 0; k--) {
            const int idx = (int)(r % p.shape[k]);
            r /= p.shape[k];
            si += idx * p.ss[k];
            di += idx * p.ds[k];
        }
        ((T *)p.dst)[di] = ((const T *)p.src)[si];
    }
}

// Transposing copies (the destination's innermost axis is strided in the source while another axis - `ya` - is the
// source's contiguous one): a 64 x 64 tile goes through shared memory so that both the reads (along ya) and the
// writes (along the innermost axis) touch consecutive addresses.  The row pitch of 64 * sizeof(T) + 4 bytes keeps the
// column reads of the store phase on distinct banks.
template <typename T>
__global__ void __launch_bounds__(256) copy_transpose_kernel(CopyParams p, int ya, long long tiles)
{
    constexpr int TILE = 64, PITCH = TILE * (int)sizeof(T) + 4;
    __shared__ __align__(16) unsigned char tile[TILE * PITCH];
    const int nx = p.shape[5], ny = p.shape[ya];
    const int tx_count = (nx + TILE - 1) / TILE, ty_count = (ny + TILE - 1) / TILE;
    for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
        long long r = t;
        const int x0 = (int)(r % tx_count) * TILE;
        r /= tx_count;
        const int y0 = (int)(r % ty_count) * TILE;
        r /= ty_count;
        long long si = 0, di = 0;
#pragma unroll
        for (int k = 4; k >= 0; k--) {
            if (k == ya)
                continue;
            const int idx = (int)(r % p.shape[k]);
            r /= p.shape[k];
            si += idx * p.ss[k];
            di += idx * p.ds[k];
        }
        const T *src = (const T *)p.src + si;
        T *dst = (T *)p.dst + di;
        __syncthreads(); // the previous tile has been stored
        {
            const int yy = threadIdx.x % TILE, xx0 = threadIdx.x / TILE;
            const T *sp = src + (long long)(x0 + xx0) * p.ss[5] + (long long)(y0 + yy) * p.ss[ya];
            const long long step = (256 / TILE) * p.ss[5];
            if (y0 + yy < ny)
                for (int xx = xx0; xx < TILE && x0 + xx < nx; xx += 256 / TILE, sp += step)
                    *(T *)(tile + xx * PITCH + yy * (int)sizeof(T)) = *sp;
        }
        __syncthreads();
        {
            const int xx = threadIdx.x % TILE, yy0 = threadIdx.x / TILE;
            T *dp = dst + (long long)(x0 + xx) * p.ds[5] + (long long)(y0 + yy0) * p.ds[ya];
            const long long step = (256 / TILE) * p.ds[ya];
            if (x0 + xx < nx)
                for (int yy = yy0; yy < TILE && y0 + yy < ny; yy += 256 / TILE, dp += step)
                    *dp = *(const T *)(tile + xx * PITCH + yy * (int)sizeof(T));
        }
    }
}

// The same tile with 32-bit global accesses: V = 4 / sizeof(T) elements per access on both sides.  The caller has checked
// that both extents, every stride that is not 1, and both pointers are multiples of V elements.
template <typename T>
__global__ void __launch_bounds__(256) copy_transpose_words_kernel(CopyParams p, int ya, long long tiles)
{
    constexpr int TILE = 64, PITCH = TILE * (int)sizeof(T) + 4, V = 4 / (int)sizeof(T), WPR = TILE / V; // words per tile row
    __shared__ __align__(16) unsigned char tile[TILE * PITCH];
    const int nx = p.shape[5], ny = p.shape[ya];
    const int tx_count = (nx + TILE - 1) / TILE, ty_count = (ny + TILE - 1) / TILE;
    for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
        long long r = t;
        const int x0 = (int)(r % tx_count) * TILE;
        r /= tx_count;
        const int y0 = (int)(r % ty_count) * TILE;
        r /= ty_count;
        long long si = 0, di = 0;
#pragma unroll
        for (int k = 4; k >= 0; k--) {
            if (k == ya)
                continue;
            const int idx = (int)(r % p.shape[k]);
            r /= p.shape[k];
            si += idx * p.ss[k];
            di += idx * p.ds[k];
        }
        const T *src = (const T *)p.src + si;
        T *dst = (T *)p.dst + di;
        __syncthreads();
        {
            const int yy = (threadIdx.x % WPR) * V, xx0 = threadIdx.x / WPR;
            const T *sp = src + (long long)(x0 + xx0) * p.ss[5] + (y0 + yy);
            const long long step = (256 / WPR) * p.ss[5];
            if (y0 + yy < ny)
                for (int xx = xx0; xx < TILE && x0 + xx < nx; xx += 256 / WPR, sp += step)
                    *(uint32_t *)(tile + xx * PITCH + yy * (int)sizeof(T)) = *(const uint32_t *)sp;
        }
        __syncthreads();
        {
            const int xx = (threadIdx.x % WPR) * V, yy0 = threadIdx.x / WPR;
            T *dp = dst + (x0 + xx) + (long long)(y0 + yy0) * p.ds[ya];
            const long long step = (256 / WPR) * p.ds[ya];
            if (x0 + xx < nx)
                for (int yy = yy0; yy < TILE && y0 + yy < ny; yy += 256 / WPR, dp += step) {
                    uint32_t w = 0;
#pragma unroll
                    for (int i = 0; i < V; i++)
                        w |= (uint32_t)(*(const T *)(tile + (xx + i) * PITCH + yy * (int)sizeof(T))) << (8 * (int)sizeof(T) * i);
                    *(uint32_t *)dp = w;
                }
        }
    }
}

// Byte transposes with 4 x 4 blocks turned in registers: a thread reads one word from each of four consecutive source rows,
// eight byte permutes give the four words of the transposed block, which go into a shared-memory tile already in
// destination order; the tile then leaves as whole words (16 bytes per thread where rows allow), 64 contiguous bytes per
// destination row.  No byte-granular shared-memory traffic on either side.  Same preconditions as the word kernel above
// (extents, strides and pointers multiples of 4).
__global__ void __launch_bounds__(256) copy_transpose_bytes4_kernel(CopyParams p, int ya, long long tiles, int vec16)
{
    constexpr int TILE = 64, PITCH = TILE + 4; // 17 words per destination row: the block stores meet two-way conflicts at most
    __shared__ __align__(16) unsigned char tile[TILE * PITCH];
    const int nx = p.shape[5], ny = p.shape[ya];
    const int tx_count = (nx + TILE - 1) / TILE, ty_count = (ny + TILE - 1) / TILE;
    for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
        long long r = t;
        const int x0 = (int)(r % tx_count) * TILE;
        r /= tx_count;
        const int y0 = (int)(r % ty_count) * TILE;
        r /= ty_count;
        long long si = 0, di = 0;
#pragma unroll
        for (int k = 4; k >= 0; k--) {
            if (k == ya)
                continue;
            const int idx = (int)(r % p.shape[k]);
            r /= p.shape[k];
            si += idx * p.ss[k];
            di += idx * p.ds[k];
        }
        const unsigned char *src = (const unsigned char *)p.src + si;
        unsigned char *dst = (unsigned char *)p.dst + di;
        __syncthreads();
        {
            // source element (x, y) lies at src + x * ss[5] + y: rows of x, contiguous along y
            const int cw = threadIdx.x & 15, g = threadIdx.x >> 4; // word of the row (4 bytes along y), group of four rows
            const int y = y0 + 4 * cw, x = x0 + 4 * g;
            if (y < ny && x < nx) {
                const unsigned char *sp = src + (long long)x * p.ss[5] + y;
                const uint32_t r0 = *(const uint32_t *)sp, r1 = *(const uint32_t *)(sp + p.ss[5]), r2 = *(const uint32_t *)(sp + 2 * p.ss[5]),
                               r3 = *(const uint32_t *)(sp + 3 * p.ss[5]);
                // bytes (r0.j, r1.j, r2.j, r3.j) -> word j
                const uint32_t a = __byte_perm(r0, r1, 0x5140), b = __byte_perm(r2, r3, 0x5140); // (r0.0 r1.0 r0.1 r1.1), (r2.0 r3.0 r2.1 r3.1)
                const uint32_t c = __byte_perm(r0, r1, 0x7362), e = __byte_perm(r2, r3, 0x7362); // (r0.2 r1.2 r0.3 r1.3), ...
                uint32_t *tp = (uint32_t *)(tile + (4 * cw) * PITCH + 4 * g);
                tp[0] = __byte_perm(a, b, 0x5410);
                tp[PITCH / 4] = __byte_perm(a, b, 0x7632);
                tp[2 * (PITCH / 4)] = __byte_perm(c, e, 0x5410);
                tp[3 * (PITCH / 4)] = __byte_perm(c, e, 0x7632);
            }
        }
        __syncthreads();
        {
            const int xq = threadIdx.x & 3, yy = threadIdx.x >> 2; // 16 bytes of one destination row
            const int y = y0 + yy, x = x0 + 16 * xq;
            if (y < ny && x < nx) {
                const uint32_t *tp = (const uint32_t *)(tile + yy * PITCH + 16 * xq);
                unsigned char *dp = dst + x + (long long)y * p.ds[ya];
                const int words = min(4, (nx - x) >> 2);
                if (vec16 && words == 4) {
                    *(uint4 *)dp = make_uint4(tp[0], tp[1], tp[2], tp[3]);
                } else {
                    for (int i = 0; i < words; i++) ((uint32_t *)dp)[i] = tp[i];
                }
            }
        }
    }
}

} // namespace espdl

using namespace espdl;

extern "C" int espdl_b200_pool(const espdl_pool_desc *d, void *stream)
{
    if (!d || !d->input || !d->output)
        return ESPDL_ERR_INVALID_ARG;
    if (d->dtype != ESPDL_DTYPE_INT8 && d->dtype != ESPDL_DTYPE_INT16)
        return ESPDL_ERR_UNSUPPORTED;
    if (d->op < ESPDL_POOL_MAX || d->op > ESPDL_POOL_GLOBAL_AVG || d->n < 0 || d->in_h <= 0 || d->in_w <= 0 || d->c <= 0)
        return ESPDL_ERR_INVALID_ARG;
    PoolParams p;
    p.in = d->input, p.out = d->output, p.op = d->op, p.is16 = d->dtype == ESPDL_DTYPE_INT16;
    p.n = d->n, p.ih = d->in_h, p.iw = d->in_w, p.c = d->c;
    if (d->op == ESPDL_POOL_GLOBAL_AVG) {
        p.oh = p.ow = 1, p.kh = d->in_h, p.kw = d->in_w, p.sh = p.sw = 1, p.pt = p.pl = 0;
    } else {
        if (d->kh <= 0 || d->kw <= 0 || d->stride_h <= 0 || d->stride_w <= 0 || d->out_h <= 0 || d->out_w <= 0)
            return ESPDL_ERR_INVALID_ARG;
        if (d->out_h != (d->in_h + d->pad_top + d->pad_bottom - d->kh) / d->stride_h + 1 ||
            d->out_w != (d->in_w + d->pad_left + d->pad_right - d->kw) / d->stride_w + 1)
            return ESPDL_ERR_INVALID_ARG;
        p.oh = d->out_h, p.ow = d->out_w, p.kh = d->kh, p.kw = d->kw, p.sh = d->stride_h, p.sw = d->stride_w;
        p.pt = d->pad_top, p.pl = d->pad_left;
    }
    if (d->in_exponent > 30 || d->in_exponent < -30 || d->out_exponent > 30 || d->out_exponent < -30)
        return ESPDL_ERR_INVALID_ARG;
    const float inv_area = 1.f / (float)(p.kh * p.kw);
    p.scale = dl_scale(d->in_exponent) * inv_area * dl_rescale(d->out_exponent);
    p.total = (long long)p.n * p.oh * p.ow * p.c;
    if (p.total == 0)
        return ESPDL_OK;
    if (d->op == ESPDL_POOL_GLOBAL_AVG && !p.is16 && p.c % 4 == 0 && ((uintptr_t)d->input % 4) == 0 && ((uintptr_t)d->output % 4) == 0) {
        const long long items = (long long)p.n * (p.c / 4);
        gap_s8_kernel<<<(unsigned)((items + 255) / 256), 256, 0, (cudaStream_t)stream>>>(p);
        count_launch();
        return check_launch("global average pool");
    }
    if (d->op == ESPDL_POOL_MAX && !p.is16 && p.c % 16 == 0 && ((uintptr_t)d->input % 16) == 0 && ((uintptr_t)d->output % 16) == 0 && p.sh == 1 &&
        p.sw == 1 && p.kh == p.kw && (p.kh == 3 || p.kh == 5) && p.oh >= 4 * p.kh && !getenv("ESPDL_B200_NO_POOL_WALK")) {
        // stride-1 windows on maps tall enough for the walk down a column to pay
        const long long columns = (long long)p.n * p.ow * (p.c / 16);
        int segments = 1; // enough threads to fill the SMs, runs of at least 2K rows
        while (columns * segments < (long long)num_sms() * 2048 && p.oh / (segments * 2) >= 2 * p.kh) segments *= 2;
        const long long items = columns * segments;
        const unsigned grid = (unsigned)min((items + 255) / 256, (long long)num_sms() * 32);
        if (p.kh == 3)
            maxpool_s8_walk_kernel<3><<<grid, 256, 0, (cudaStream_t)stream>>>(p, segments);
        else
            maxpool_s8_walk_kernel<5><<<grid, 256, 0, (cudaStream_t)stream>>>(p, segments);
        count_launch();
        return check_launch("max pool walk");
    }
    if (d->op == ESPDL_POOL_MAX && !p.is16 && p.c % 16 == 0 && ((uintptr_t)d->input % 16) == 0 && ((uintptr_t)d->output % 16) == 0) {
        const long long items = p.total / 16;
        maxpool_s8_vec16_kernel<<<(unsigned)min((items + 255) / 256, (long long)num_sms() * 32), 256, 0, (cudaStream_t)stream>>>(p);
        count_launch();
        return check_launch("max pool");
    }
    long long blocks = min((p.total + 255) / 256, (long long)num_sms() * 32);
    pool_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
    count_launch();
    return check_launch("pool");
}

// Linear resize (esp-dl/dl/base/dl_base_resize.cpp:80-236): source coordinate and the two weights per axis as
// linear_coeffs computes them, products and sums rounded one by one in fp32 (no fused multiply-add), then
// quantize = clip(round(v * 2^-e_out)).
struct ResizeLinearParams {
    const int8_t *in;
    int8_t *out;
    int n, ih, iw, c, oh, ow, ops, align, one_d;
    float sh_inv, sw_inv, in_scale, out_rescale;
    long long total;
};

__device__ __forceinline__ void linear_coeffs_dev(int o, int &i, float &r0, float &r1, int in_length, float scale_inv, int align)
{
    float fx = align ? __fmul_rn((float)o, scale_inv) : __fsub_rn(__fmul_rn(__fadd_rn((float)o, 0.5f), scale_inv), 0.5f);
    i = (int)floorf(fx);
    fx = __fsub_rn(fx, (float)i);
    if (i < 0) {
        i = 0;
        fx = 0.f;
    }
    if (i >= in_length - 1) {
        i = in_length - 2;
        fx = 1.f;
    }
    r0 = __fsub_rn(1.f, fx);
    r1 = fx;
}

__global__ void __launch_bounds__(256) resize_linear_kernel(ResizeLinearParams p)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < p.total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % p.c);
        const long long pix = i / p.c;
        const int x = (int)(pix % p.ow);
        const int y = (int)((pix / p.ow) % p.oh);
        const int n = (int)(pix / ((long long)p.ow * p.oh));
        int ix, iy = 0;
        float xr0, xr1, yr0 = 1.f, yr1 = 0.f;
        linear_coeffs_dev(x, ix, xr0, xr1, p.iw, p.sw_inv, p.align);
        if (!p.one_d)
            linear_coeffs_dev(y, iy, yr0, yr1, p.ih, p.sh_inv, p.align);
        const int8_t *row0 = p.in + (((long long)n * p.ih + iy) * p.iw + ix) * p.c + c;
        const float a0 = __fmul_rn((float)row0[0], p.in_scale), a1 = __fmul_rn((float)row0[p.c], p.in_scale);
        float v = __fadd_rn(__fmul_rn(a0, xr0), __fmul_rn(a1, xr1));
        if (!p.one_d) {
            const int8_t *row1 = row0 + (long long)p.iw * p.c;
            const float b0 = __fmul_rn((float)row1[0], p.in_scale), b1 = __fmul_rn((float)row1[p.c], p.in_scale);
            const float w = __fadd_rn(__fmul_rn(b0, xr0), __fmul_rn(b1, xr1));
            v = __fadd_rn(__fmul_rn(v, yr0), __fmul_rn(w, yr1));
        }
        p.out[pix * p.ops + c] = (int8_t)sat8(fround_half_up(__fmul_rn(v, p.out_rescale)));
    }
}

extern "C" int espdl_b200_resize(const espdl_resize_desc *d, void *stream)
{
    if (!d || !d->input || !d->output)
        return ESPDL_ERR_INVALID_ARG;
    if (d->dtype != ESPDL_DTYPE_INT8) // the reference's int16 resize is an empty function (dl_base_resize.cpp:298-309)
        return ESPDL_ERR_UNSUPPORTED;
    if (d->n < 0 || d->in_h <= 0 || d->in_w <= 0 || d->c <= 0 || d->out_h <= 0 || d->out_w <= 0 || d->scale_h <= 0 || d->scale_w <= 0)
        return ESPDL_ERR_INVALID_ARG;
    if (d->mode < 0 || d->mode > 2)
        return ESPDL_ERR_INVALID_ARG;
    if (d->mode != 0) {
        ResizeLinearParams q;
        q.in = (const int8_t *)d->input, q.out = (int8_t *)d->output;
        q.n = d->n, q.ih = d->in_h, q.iw = d->in_w, q.c = d->c, q.oh = d->out_h, q.ow = d->out_w;
        q.ops = d->out_pixel_stride ? d->out_pixel_stride : d->c;
        q.align = d->mode == 2, q.one_d = d->in_h == 1 && d->out_h == 1;
        if (d->in_w < 2 || (!q.one_d && d->in_h < 2) || abs(d->in_exponent) > 30 || abs(d->out_exponent) > 30)
            return ESPDL_ERR_UNSUPPORTED;
        float sh = d->scale_h, sw = d->scale_w;
        if (q.align) { // dl_base_resize.hpp:46-62
            sh = q.one_d ? 1.f : (d->out_h - 1) / (float)(d->in_h - 1);
            sw = (d->out_w - 1) / (float)(d->in_w - 1);
        }
        q.sh_inv = 1 / sh, q.sw_inv = 1 / sw;
        q.in_scale = dl_scale(d->in_exponent), q.out_rescale = dl_rescale(d->out_exponent);
        q.total = (long long)q.n * q.oh * q.ow * q.c;
        if (q.total == 0)
            return ESPDL_OK;
        resize_linear_kernel<<<(unsigned)min((q.total + 255) / 256, (long long)num_sms() * 32), 256, 0, (cudaStream_t)stream>>>(q);
        count_launch();
        return check_launch("resize_linear");
    }
    ResizeParams p;
    p.in = (const int8_t *)d->input, p.out = (int8_t *)d->output;
    p.n = d->n, p.ih = d->in_h, p.iw = d->in_w, p.c = d->c, p.oh = d->out_h, p.ow = d->out_w;
    p.ops = d->out_pixel_stride ? d->out_pixel_stride : d->c;
    p.two = d->scale_h == 2 && d->scale_w == 2;
    p.sh_inv = 1 / d->scale_h, p.sw_inv = 1 / d->scale_w;
    int shift = d->out_exponent - d->in_exponent, oscale = 1;
    if (shift < 0) {
        oscale = 1 << (-shift);
        shift = 0;
    }
    if (shift > 30 || oscale > (1 << 30))
        return ESPDL_ERR_INVALID_ARG;
    p.oscale = (float)oscale, p.odiv = (float)(1 << shift);
    p.total = (long long)p.n * p.oh * p.ow * p.c;
    if (p.total == 0)
        return ESPDL_OK;
    if (oscale == 1 && shift == 0 && p.c % 16 == 0 && p.ops % 16 == 0 && ((uintptr_t)d->input % 16) == 0 && ((uintptr_t)d->output % 16) == 0) {
        const long long items = p.total / 16;
        resize_nearest_vec16_kernel<<<(unsigned)min((items + 255) / 256, (long long)num_sms() * 32), 256, 0, (cudaStream_t)stream>>>(p);
        count_launch();
        return check_launch("resize");
    }
    long long blocks = min((p.total + 255) / 256, (long long)num_sms() * 32);
    resize_nearest_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
    count_launch();
    return check_launch("resize");
}

// Gather along one axis (dl_module_gather.hpp:66-96): rows of `inner` elements picked by index.  A thread moves one
// unit of the row: 16 bytes when rows and pointers allow it, else one element.
template <typename U>
__global__ void __launch_bounds__(256) gather_kernel(const U *in, U *out, const int *indices, int num, long long outer, long long axis, long long inner)
{
    const long long total = outer * num * inner;
    for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
        const long long col = t % inner, row = t / inner;
        const int idx = indices[row % num];
        if (idx >= 0 && idx < axis)
            out[t] = in[((row / num) * axis + idx) * inner + col];
    }
}

extern "C" int espdl_b200_gather(const espdl_gather_desc *d, void *stream)
{
    if (!d || !d->input || !d->output || !d->indices || d->num_indices < 0 || d->outer < 0 || d->axis_size <= 0 || d->inner < 0)
        return ESPDL_ERR_INVALID_ARG;
    if (d->elem_size != 1 && d->elem_size != 2 && d->elem_size != 4 && d->elem_size != 8)
        return ESPDL_ERR_INVALID_ARG;
    long long inner = d->inner;
    int es = d->elem_size;
    if (d->outer * d->num_indices * inner == 0)
        return ESPDL_OK;
    while (es < 16 && inner % 2 == 0 && ((uintptr_t)d->input % (es * 2)) == 0 && ((uintptr_t)d->output % (es * 2)) == 0) inner /= 2, es *= 2;
    const long long total = d->outer * d->num_indices * inner;
    const unsigned blocks = (unsigned)min((total + 255) / 256, (long long)num_sms() * 32);
    cudaStream_t s = (cudaStream_t)stream;
    switch (es) {
    case 1: gather_kernel<uint8_t><<<blocks, 256, 0, s>>>((const uint8_t *)d->input, (uint8_t *)d->output, d->indices, d->num_indices, d->outer, d->axis_size, inner); break;
    case 2: gather_kernel<uint16_t><<<blocks, 256, 0, s>>>((const uint16_t *)d->input, (uint16_t *)d->output, d->indices, d->num_indices, d->outer, d->axis_size, inner); break;
    case 4: gather_kernel<uint32_t><<<blocks, 256, 0, s>>>((const uint32_t *)d->input, (uint32_t *)d->output, d->indices, d->num_indices, d->outer, d->axis_size, inner); break;
    case 8: gather_kernel<uint2><<<blocks, 256, 0, s>>>((const uint2 *)d->input, (uint2 *)d->output, d->indices, d->num_indices, d->outer, d->axis_size, inner); break;
    default: gather_kernel<uint4><<<blocks, 256, 0, s>>>((const uint4 *)d->input, (uint4 *)d->output, d->indices, d->num_indices, d->outer, d->axis_size, inner); break;
    }
    count_launch();
    return check_launch("gather");
}

// Concat / Split in one launch: a thread moves one 16-byte unit of a row of the wide tensor; which part the unit
// belongs to comes from a table of at most eight unit offsets.
namespace espdl {
namespace {
struct PartsParams {
    uint4 *wide;
    uint4 *parts[8];
    int start[9]; // first unit of part i inside a row of the wide tensor; start[n_parts] = units per row
    long long pitch[8]; // units between rows of part i; a null part is left alone
    int n_parts, split;
    long long total; // rows x units per row
};

__global__ void __launch_bounds__(256) concat_split_kernel(PartsParams p)
{
    const int upr = p.start[p.n_parts];
    for (long long u = blockIdx.x * (long long)blockDim.x + threadIdx.x; u < p.total; u += (long long)gridDim.x * blockDim.x) {
        const long long row = u / upr;
        const int col = (int)(u - row * upr);
        int i = 0;
#pragma unroll
        for (int k = 1; k < 8; k++)
            if (k < p.n_parts && col >= p.start[k])
                i = k;
        if (!p.parts[i])
            continue;
        uint4 *part = p.parts[i] + row * p.pitch[i] + (col - p.start[i]);
        if (p.split)
            *part = p.wide[u];
        else
            p.wide[u] = *part;
    }
}
} // namespace
} // namespace espdl

extern "C" int espdl_b200_concat_split(const espdl_parts_desc *d, void *stream)
{
    if (!d || !d->wide || d->n_parts < 1 || d->n_parts > 8 || d->rows < 0 || ((uintptr_t)d->wide % 16))
        return ESPDL_ERR_INVALID_ARG;
    PartsParams p;
    p.wide = (uint4 *)d->wide, p.n_parts = d->n_parts, p.split = d->split ? 1 : 0;
    long long units = 0;
    for (int i = 0; i < 8; i++) {
        p.parts[i] = nullptr;
        p.start[i] = (int)units;
        p.pitch[i] = 0;
        if (i < d->n_parts) {
            if (d->part_bytes[i] <= 0 || d->part_bytes[i] % 16)
                return ESPDL_ERR_INVALID_ARG;
            if (!d->skip[i]) {
                if (!d->parts[i] || ((uintptr_t)d->parts[i] % 16) || d->part_stride[i] % 16 || (d->part_stride[i] && d->part_stride[i] < d->part_bytes[i]))
                    return ESPDL_ERR_INVALID_ARG;
                p.parts[i] = (uint4 *)d->parts[i];
                p.pitch[i] = (d->part_stride[i] ? d->part_stride[i] : d->part_bytes[i]) / 16;
            }
            units += d->part_bytes[i] / 16;
            if (units > 0x7fffffffll)
                return ESPDL_ERR_TOO_LARGE;
        }
    }
    for (int i = d->n_parts; i <= 8; i++) p.start[i] = (int)units;
    p.total = d->rows * units;
    if (p.total == 0)
        return ESPDL_OK;
    const long long blocks = (p.total + 255) / 256;
    concat_split_kernel<<<(unsigned)min(blocks, (long long)num_sms() * 32), 256, 0, (cudaStream_t)stream>>>(p);
    count_launch();
    return check_launch("concat_split");
}

extern "C" int espdl_b200_copy(const espdl_copy_desc *d, void *stream)
{
    if (!d || !d->src || !d->dst || d->ndim < 1 || d->ndim > 6)
        return ESPDL_ERR_INVALID_ARG;
    if (d->elem_size != 1 && d->elem_size != 2 && d->elem_size != 4 && d->elem_size != 8)
        return ESPDL_ERR_INVALID_ARG;
    CopyParams p;
    p.src = (const char *)d->src, p.dst = (char *)d->dst, p.es = d->elem_size;
    p.total = 1;
    for (int i = 0; i < 6; i++) p.shape[i] = 1, p.ss[i] = 0, p.ds[i] = 0;
    for (int i = 0; i < d->ndim; i++) {
        if (d->shape[i] < 0)
            return ESPDL_ERR_INVALID_ARG;
        p.shape[6 - d->ndim + i] = d->shape[i];
        p.ss[6 - d->ndim + i] = d->src_stride[i];
        p.ds[6 - d->ndim + i] = d->dst_stride[i];
        p.total *= d->shape[i];
    }
    if (p.total == 0)
        return ESPDL_OK;
    // widen the element when the innermost run is contiguous and everything is aligned
    int es = d->elem_size;
    while (es < 16) {
        const int f = 2;
        bool ok = p.ss[5] == 1 && p.ds[5] == 1 && p.shape[5] % f == 0 && ((uintptr_t)p.src % (es * f)) == 0 && ((uintptr_t)p.dst % (es * f)) == 0;
        for (int k = 0; k < 5 && ok; k++) ok = p.ss[k] % f == 0 && p.ds[k] % f == 0;
        if (!ok)
            break;
        p.shape[5] /= f;
        for (int k = 0; k < 5; k++) p.ss[k] /= f, p.ds[k] /= f;
        p.total /= f;
        es *= f;
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (es <= 2 && p.ds[5] == 1 && p.ss[5] != 1 && p.shape[5] >= 16) {
        int ya = -1;
        for (int k = 4; k >= 0; k--)
            if (p.ss[k] == 1 && p.shape[k] >= 16)
                ya = k;
        if (ya >= 0) {
            long long tiles = (long long)((p.shape[5] + 63) / 64) * ((p.shape[ya] + 63) / 64);
            for (int k = 0; k < 5; k++)
                if (k != ya)
                    tiles *= p.shape[k];
            const unsigned grid = (unsigned)min(tiles, (long long)num_sms() * 16);
            const int V = 4 / es;
            bool words = p.shape[5] % V == 0 && p.shape[ya] % V == 0 && ((uintptr_t)p.src % 4) == 0 && ((uintptr_t)p.dst % 4) == 0;
            for (int k = 0; k < 6 && words; k++) {
                if (k != ya && p.shape[k] > 1 && p.ss[k] % V != 0)
                    words = false; // source rows start on word boundaries
                if (k != 5 && p.shape[k] > 1 && p.ds[k] % V != 0)
                    words = false;
            }
            if (words && es == 1 && !getenv("ESPDL_B200_NO_TRANSPOSE4")) {
                // 16-byte stores when every destination row starts on a 16-byte boundary
                bool vec16 = ((uintptr_t)p.dst % 16) == 0;
                for (int k = 0; k < 5 && vec16; k++)
                    if (p.shape[k] > 1 && p.ds[k] % 16 != 0)
                        vec16 = false;
                copy_transpose_bytes4_kernel<<<grid, 256, 0, s>>>(p, ya, tiles, vec16 ? 1 : 0);
            } else if (words && es == 1)
                copy_transpose_words_kernel<uint8_t><<<grid, 256, 0, s>>>(p, ya, tiles);
            else if (words)
                copy_transpose_words_kernel<uint16_t><<<grid, 256, 0, s>>>(p, ya, tiles);
            else if (es == 1)
                copy_transpose_kernel<uint8_t><<<grid, 256, 0, s>>>(p, ya, tiles);
            else
                copy_transpose_kernel<uint16_t><<<grid, 256, 0, s>>>(p, ya, tiles);
            count_launch();
            return check_launch("copy");
        }
    }
    long long blocks = min((p.total + 255) / 256, (long long)num_sms() * 32);
    switch (es) {
    case 1: copy_kernel<uint8_t><<<(unsigned)blocks, 256, 0, s>>>(p); break;
    case 2: copy_kernel<uint16_t><<<(unsigned)blocks, 256, 0, s>>>(p); break;
    case 4: copy_kernel<uint32_t><<<(unsigned)blocks, 256, 0, s>>>(p); break;
    case 8: copy_kernel<uint2><<<(unsigned)blocks, 256, 0, s>>>(p); break;
    default: copy_kernel<uint4><<<(unsigned)blocks, 256, 0, s>>>(p); break;
    }
    count_launch();
    return check_launch("copy");
}
