// Int8 2-D convolution (NHWC, filter [outC, kH, kW, inC/group]) for Glow's
// ChannelwiseQuantizedConvolution and quantized Convolution.
//
// group == 1: the convolution is the int8 contraction of qgemm.cu over an im2col matrix
//   A[n*OH*OW + oh*OW + ow, (kh*KW + kw)*C + c] = X[n, oh*SH - PT + kh*DH, ow*SW - PL + kw*DW, c]
// whose result rows are exactly the NHWC output.  Taps outside the image are skipped by the
// reference (libjit_conv.cpp:209-212), i.e. they contribute (x - inOffset) = 0: im2col writes
// inOffset there.  The filter [outC, kH*kW*C] already is the K-major right-hand side.  A 1x1,
// stride-1, unpadded convolution needs no im2col at all.  When kH*kW*C is not a multiple of 16
// both operands are padded with zeros along K (zeros add nothing to the raw products or to the
// row sums; the offset correction uses the true K).
// group > 1 (and anything else unusual): a direct kernel, one thread per output, the
// reference's loop nest as written.
#include "common.cuh"
#include "qgemm.cuh"

// 1: stride-1 windows take the shifted-rows path (no im2col matrix) when the shapes allow
#ifndef GLOWB200_CONV_SHIFTED_ROWS
#define GLOWB200_CONV_SHIFTED_ROWS 1
#endif

namespace glowb200 {
namespace {

struct ConvGeom {
  int N, H, W, C, OH, OW, OC, KH, KW, SH, SW, PT, PL, DH, DW, G;
};

// one thread per 16-byte chunk of the im2col matrix (C a multiple of 16: a chunk never
// straddles two taps)
__global__ void __launch_bounds__(256) im2col_i8_vec_kernel(const int8_t *__restrict__ x, int8_t *__restrict__ a,
                                                             const __grid_constant__ ConvGeom g, int Kpad, int pad_word) {
  pdl_wait();
  pdl_launch_dependents();
  const int chunks_per_row = Kpad >> 4;
  const int64_t total = (int64_t)g.N * g.OH * g.OW * chunks_per_row;
  const int c_chunks = g.C >> 4;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / chunks_per_row;
    const int ch = (int)(i - row * chunks_per_row);
    const int tap = ch / c_chunks, cc = ch - tap * c_chunks;
    int4 v = make_int4(0, 0, 0, 0);
    if (tap < g.KH * g.KW) {
      const int kh = tap / g.KW, kw = tap - kh * g.KW;
      const int ow = (int)(row % g.OW);
      const int64_t r2 = row / g.OW;
      const int oh = (int)(r2 % g.OH), n = (int)(r2 / g.OH);
      const int ih = oh * g.SH - g.PT + kh * g.DH, iw = ow * g.SW - g.PL + kw * g.DW;
      if (ih >= 0 && iw >= 0 && ih < g.H && iw < g.W)
        v = *reinterpret_cast<const int4 *>(x + (((int64_t)n * g.H + ih) * g.W + iw) * g.C + cc * 16);
      else
        v = make_int4(pad_word, pad_word, pad_word, pad_word);
    }
    *reinterpret_cast<int4 *>(a + row * Kpad + ch * 16) = v;
  }
}

// any channel count: one thread per byte
__global__ void __launch_bounds__(256) im2col_i8_kernel(const int8_t *__restrict__ x, int8_t *__restrict__ a,
                                                         const __grid_constant__ ConvGeom g, int K, int Kpad, int8_t pad) {
  const int64_t total = (int64_t)g.N * g.OH * g.OW * Kpad;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / Kpad;
    const int k = (int)(i - row * Kpad);
    int8_t v = 0;
    if (k < K) {
      const int tap = k / g.C, c = k - tap * g.C;
      const int kh = tap / g.KW, kw = tap - kh * g.KW;
      const int ow = (int)(row % g.OW);
      const int64_t r2 = row / g.OW;
      const int oh = (int)(r2 % g.OH), n = (int)(r2 / g.OH);
      const int ih = oh * g.SH - g.PT + kh * g.DH, iw = ow * g.SW - g.PL + kw * g.DW;
      v = (ih >= 0 && iw >= 0 && ih < g.H && iw < g.W) ? x[(((int64_t)n * g.H + ih) * g.W + iw) * g.C + c] : pad;
    }
    a[i] = v;
  }
}

// Bytes of a staged input row of im2col_i8_rows_kernel: the image row, its left padding and as much
// on the right as the last output pixel's window reaches.
__host__ __device__ inline int64_t rows_pitch(const ConvGeom &g) {
  const int64_t last = (int64_t)(g.OW - 1) * g.SW + (int64_t)(g.KW - 1) * g.DW + 1;  // pixels from the padded row's start
  const int64_t have = (int64_t)g.PL + g.W;
  return (last > have ? last : have) * g.C;
}

// Any channel count, one block per output image row (n, oh).  The KH input rows the image row
// needs are staged in shared memory with their horizontal padding made real (`pad` left and right
// of the image, whole rows of it above and below), so a tap is a plain offset from the pixel's
// window.  A thread keeps ONE 16-byte piece of the im2col row (piece = thread % pieces per row) for
// all the pixels it visits: the sixteen offsets of its bytes are worked out once, and a piece then
// costs sixteen byte loads, the packing and one vector store.  (Walking (kh, kw, c) with counters
// for every piece, as this kernel first did, took 163 us for a 7 x 7 stride-2 stem over 3 channels
// at batch 64: about 170 instructions per 16 bytes.)
// Shared memory: KH rows of `pitch` bytes (checked by the launcher).
__global__ void __launch_bounds__(256) im2col_i8_rows_kernel(const int8_t *__restrict__ x, int8_t *__restrict__ a,
                                                              const __grid_constant__ ConvGeom g, int K, int Kpad, int8_t pad,
                                                              int pitch) {
  extern __shared__ __align__(16) int8_t rows_smem[];
  const int n = blockIdx.x / g.OH, oh = blockIdx.x - n * g.OH;
  const int row_bytes = g.W * g.C, left = g.PL * g.C;
  for (int kh = 0; kh < g.KH; kh++) {
    const int ih = oh * g.SH - g.PT + kh * g.DH;
    int8_t *dst = rows_smem + kh * pitch;
    if (ih < 0 || ih >= g.H) {
      for (int j = threadIdx.x; j < pitch; j += blockDim.x) dst[j] = pad;
      continue;
    }
    const int8_t *src = x + ((int64_t)n * g.H + ih) * row_bytes;
    for (int j = threadIdx.x; j < pitch - row_bytes; j += blockDim.x) dst[j < left ? j : j + row_bytes] = pad;
    if (((reinterpret_cast<uintptr_t>(src) | (uintptr_t)row_bytes) & 3) == 0) {
      for (int j = threadIdx.x * 4; j < row_bytes; j += blockDim.x * 4) {
        const uint32_t v = __ldg(reinterpret_cast<const uint32_t *>(src + j));
        dst[left + j] = (int8_t)v;
        dst[left + j + 1] = (int8_t)(v >> 8);
        dst[left + j + 2] = (int8_t)(v >> 16);
        dst[left + j + 3] = (int8_t)(v >> 24);
      }
    } else {
      for (int j = threadIdx.x; j < row_bytes; j += blockDim.x) dst[left + j] = src[j];
    }
  }
  const int pieces = Kpad >> 4;
  const int ch = threadIdx.x % pieces, slot = threadIdx.x / pieces, slots = blockDim.x / pieces;
  int off[16];
  uint32_t keep[4] = {0u, 0u, 0u, 0u};  // bytes of the piece that are taps (the rest is the zero padding of K)
#pragma unroll
  for (int b = 0; b < 16; b++) {
    const int k = ch * 16 + b;
    off[b] = 0;
    if (k < K) {
      const int tap = k / g.C, c = k - tap * g.C;
      const int kh = tap / g.KW, kw = tap - kh * g.KW;
      off[b] = kh * pitch + kw * g.DW * g.C + c;
      keep[b >> 2] |= 0xffu << (8 * (b & 3));
    }
  }
  __syncthreads();
  int8_t *out = a + ((int64_t)n * g.OH + oh) * g.OW * Kpad + ch * 16;
  if (slot < slots) {
    for (int ow = slot; ow < g.OW; ow += slots) {
      const uint8_t *win = reinterpret_cast<const uint8_t *>(rows_smem) + ow * g.SW * g.C;
      uint32_t w[4];
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const uint32_t lo = __byte_perm(win[off[4 * q]], win[off[4 * q + 1]], 0x0040);
        const uint32_t hi = __byte_perm(win[off[4 * q + 2]], win[off[4 * q + 3]], 0x0040);
        w[q] = __byte_perm(lo, hi, 0x5410) & keep[q];
      }
      *reinterpret_cast<int4 *>(out + (int64_t)ow * Kpad) = make_int4((int)w[0], (int)w[1], (int)w[2], (int)w[3]);
    }
  }
}

// Row windows of a stride-2 convolution over few channels (KW * C <= 32, no dilation): plane e
// (e = 0, 1), image n, row y, output column ow holds the KW * C bytes x[n, 2y - PT + e, 2ow - PL .. + KW - 1, :]
// and zeros up to 32 bytes; cells outside the image hold `pad` (the input offset).  Tap (kh = 2a + e, kw)
// of output pixel (n, oh, ow) is byte kw * C + c of window (n, oh + a, ow) of plane e, so the
// convolution is a contraction whose left-hand rows are four windows of one plane, Y = OH + 3 rows
// per image: 2 * 32 bytes per (y, ow) instead of KH * KW * C per output pixel, and no im2col matrix.
// One thread per window.
__global__ void __launch_bounds__(256) row_windows_i8_kernel(const int8_t *__restrict__ x, int8_t *__restrict__ planes,
                                                              const __grid_constant__ ConvGeom g, int Y, int64_t plane_bytes,
                                                              int8_t pad) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t per_plane = (int64_t)g.N * Y * g.OW, total = 2 * per_plane;
  const int run = g.KW * g.C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int e = (int)(i / per_plane);
    int64_t r = i - e * per_plane;
    const int ow = (int)(r % g.OW);
    r /= g.OW;
    const int y = (int)(r % Y), n = (int)(r / Y);
    const int ih = 2 * y - g.PT + e, b0 = (2 * ow - g.PL) * g.C;  // first byte of the window in its image row
    const bool row_in = ih >= 0 && ih < g.H;
    const int8_t *src = x + ((int64_t)n * g.H + (row_in ? ih : 0)) * g.W * g.C;
    uint32_t w[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    for (int b = 0; b < run; b++) {
      const int o = b0 + b;
      const int8_t v = (row_in && o >= 0 && o < g.W * g.C) ? src[o] : pad;
      w[b >> 2] |= (uint32_t)(uint8_t)v << (8 * (b & 3));
    }
    int4 *dst = reinterpret_cast<int4 *>(planes + e * plane_bytes + (i - e * per_plane) * 32);
    dst[0] = make_int4((int)w[0], (int)w[1], (int)w[2], (int)w[3]);
    dst[1] = make_int4((int)w[4], (int)w[5], (int)w[6], (int)w[7]);
  }
}

// Filter [OC, KH, KW, C] -> [OC, 2 planes, 4 rows a, 32 bytes]: tap (kh = 2a + e, kw, c) at byte
// kw * C + c of (e, a); everything else zero.
__global__ void __launch_bounds__(256) window_filter_i8_kernel(const int8_t *__restrict__ f, int8_t *__restrict__ out, int OC,
                                                               int KH, int KW, int C) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t total = (int64_t)OC * 256;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int oc = (int)(i >> 8), k = (int)(i & 255);
    const int e = k >> 7, a = (k >> 5) & 3, b = k & 31;
    const int kh = 2 * a + e, kw = b / C, c = b - kw * C;
    out[i] = (kh < KH && kw < KW) ? f[(((int64_t)oc * KH + kh) * KW + kw) * C + c] : (int8_t)0;
  }
}

// NHWC input with its padding made real: [N, Hp, Wp, C], the cells outside the image filled with
// `pad_word` (the input offset, which is how the reference's skipped taps read).  16 bytes per thread.
__global__ void __launch_bounds__(256) pad_nhwc_i8_kernel(const int8_t *__restrict__ x, int8_t *__restrict__ xp,
                                                           const __grid_constant__ ConvGeom g, int Hp, int Wp, int pad_word) {
  pdl_wait();
  pdl_launch_dependents();
  const int cc = g.C >> 4;
  const int64_t total = (int64_t)g.N * Hp * Wp * cc;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % cc);
    int64_t r = i / cc;
    const int xw = (int)(r % Wp);
    r /= Wp;
    const int yh = (int)(r % Hp), n = (int)(r / Hp);
    const int ih = yh - g.PT, iw = xw - g.PL;
    int4 v = make_int4(pad_word, pad_word, pad_word, pad_word);
    if (ih >= 0 && iw >= 0 && ih < g.H && iw < g.W)
      v = __ldg(reinterpret_cast<const int4 *>(x + (((int64_t)n * g.H + ih) * g.W + iw) * g.C) + c);
    reinterpret_cast<int4 *>(xp)[i] = v;
  }
}

// The same for a stride-2 window, split by the parity of the padded coordinates: plane (ph, pw) holds
// the padded input at (2y + ph, 2x + pw), [4][N, Hq, Wq, C].  Tap (kh, kw) of output pixel (n, oh, ow)
// is then pixel (n, oh + kh / 2, ow + kw / 2) of plane (kh & 1, kw & 1): a row offset again.
__global__ void __launch_bounds__(256) pad_parity_nhwc_i8_kernel(const int8_t *__restrict__ x, int8_t *__restrict__ xp,
                                                                  const __grid_constant__ ConvGeom g, int Hq, int Wq, int pad_word) {
  pdl_wait();
  pdl_launch_dependents();
  const int cc = g.C >> 4;
  const int64_t total = 4ll * g.N * Hq * Wq * cc;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % cc);
    int64_t r = i / cc;
    const int xq = (int)(r % Wq);
    r /= Wq;
    const int yq = (int)(r % Hq);
    r /= Hq;
    const int n = (int)(r % g.N), plane = (int)(r / g.N);
    const int ih = 2 * yq + (plane >> 1) - g.PT, iw = 2 * xq + (plane & 1) - g.PL;
    int4 v = make_int4(pad_word, pad_word, pad_word, pad_word);
    if (ih >= 0 && iw >= 0 && ih < g.H && iw < g.W)
      v = __ldg(reinterpret_cast<const int4 *>(x + (((int64_t)n * g.H + ih) * g.W + iw) * g.C) + c);
    reinterpret_cast<int4 *>(xp)[i] = v;
  }
}

// Filter [OC, KH, KW, 64] -> [OC, KH * ceil(KW / 2), 128]: taps (kh, 2j) and (kh, 2j + 1) side by
// side, the partner of a last odd tap zero -- the right-hand side that matches left-hand rows made of
// two neighbouring 64-channel pixels.
__global__ void __launch_bounds__(256) pair_taps_c64_kernel(const int8_t *__restrict__ f, int8_t *__restrict__ out, int OC,
                                                             int KH, int KW) {
  pdl_wait();
  pdl_launch_dependents();
  const int pairs = (KW + 1) >> 1;
  const int64_t total = (int64_t)OC * KH * pairs * 128;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int j = (int)(i & 127);
    int64_t r = i >> 7;
    const int pr = (int)(r % pairs);
    r /= pairs;
    const int kh = (int)(r % KH), oc = (int)(r / KH);
    const int kw = 2 * pr + (j >> 6);
    out[i] = kw < KW ? f[(((int64_t)oc * KH + kh) * KW + kw) * 64 + (j & 63)] : (int8_t)0;
  }
}

// [rows, K] -> [rows, Kpad], zero padded
__global__ void __launch_bounds__(256) pad_rows_i8_kernel(const int8_t *__restrict__ in, int8_t *__restrict__ out, int rows,
                                                           int K, int Kpad) {
  const int64_t total = (int64_t)rows * Kpad;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / Kpad;
    const int k = (int)(i - r * Kpad);
    out[i] = k < K ? in[r * K + k] : (int8_t)0;
  }
}

// The reference's loop nest (libjit_conv.cpp:151-239 / :49-147), one thread per output element.
__global__ void __launch_bounds__(256) conv2d_i8_direct_kernel(const int8_t *__restrict__ x, const int8_t *__restrict__ f,
                                                                const __grid_constant__ ConvGeom g,
                                                                const __grid_constant__ GemmParams p) {
  const int64_t total = (int64_t)g.N * g.OH * g.OW * g.OC;
  const int icg = g.C / g.G, ocg = g.OC / g.G;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(i % g.OC);
    int64_t r = i / g.OC;
    const int ow = (int)(r % g.OW);
    r /= g.OW;
    const int oh = (int)(r % g.OH), n = (int)(r / g.OH);
    const int grp = d / ocg;
    const ColQuant q = col_quant(p, d);
    uint32_t sum = (uint32_t)scale32(load_bias(p, d) - (p.bias_offsets ? p.bias_offsets[d] : p.bias_offset), q.bias_pre,
                                     q.bias_post, q.bias_scale, 0);
    for (int kh = 0; kh < g.KH; kh++)
      for (int kw = 0; kw < g.KW; kw++) {
        const int ih = oh * g.SH - g.PT + kh * g.DH, iw = ow * g.SW - g.PL + kw * g.DW;
        if (ih < 0 || iw < 0 || ih >= g.H || iw >= g.W) continue;
        const int8_t *xp = x + (((int64_t)n * g.H + ih) * g.W + iw) * g.C + grp * icg;
        const int8_t *fp = f + (((int64_t)d * g.KH + kh) * g.KW + kw) * icg;
        for (int c = 0; c < icg; c++) sum += (uint32_t)(((int32_t)fp[c] - q.b_off) * ((int32_t)xp[c] - p.a_offset));
      }
    p.out[i] = (int8_t)clip_i8(activation_i32(scale32((int32_t)sum, q.out_pre, q.out_post, q.out_scale, p.out_offset), p));
  }
}

int geom_from_dims(ConvGeom &g, const int64_t *out_dims, const int64_t *in_dims, const int64_t *filter_dims,
                   const int64_t *kernels, const int64_t *strides, const int64_t *pads, int64_t group,
                   const int64_t *dilation) {
  GLOWB200_REQUIRE(out_dims && in_dims && filter_dims && kernels && strides && pads && dilation, "NULL shape array");
  for (int i = 0; i < 4; i++)
    GLOWB200_REQUIRE(out_dims[i] >= 0 && in_dims[i] >= 0 && filter_dims[i] >= 0 && out_dims[i] < (1ll << 31) &&
                         in_dims[i] < (1ll << 31) && filter_dims[i] < (1ll << 31), "dimension out of range");
  g.N = (int)in_dims[0]; g.H = (int)in_dims[1]; g.W = (int)in_dims[2]; g.C = (int)in_dims[3];
  g.OH = (int)out_dims[1]; g.OW = (int)out_dims[2]; g.OC = (int)out_dims[3];
  g.KH = (int)kernels[0]; g.KW = (int)kernels[1];
  g.SH = (int)strides[0]; g.SW = (int)strides[1];
  g.PT = (int)pads[0]; g.PL = (int)pads[1];
  g.DH = (int)dilation[0]; g.DW = (int)dilation[1];
  g.G = (int)group;
  GLOWB200_REQUIRE(out_dims[0] == in_dims[0], "batch sizes of input and output differ");
  GLOWB200_REQUIRE(g.G >= 1 && g.C % g.G == 0 && g.OC % g.G == 0, "channels not divisible by the group count");
  GLOWB200_REQUIRE(filter_dims[0] == g.OC && filter_dims[1] == g.KH && filter_dims[2] == g.KW &&
                       filter_dims[3] == g.C / g.G, "filter dims do not match [outC, kH, kW, inC/group]");
  GLOWB200_REQUIRE(g.SH >= 1 && g.SW >= 1 && g.DH >= 1 && g.DW >= 1 && g.KH >= 1 && g.KW >= 1, "bad stride/dilation/kernel");
  return GLOWB200_OK;
}

struct ConvPlan {
  bool direct;       // direct kernel (groups, empty)
  bool need_im2col;  // else the input itself is the left-hand side
  int K, Kpad;
  int64_t M;
  size_t a_bytes, f_bytes, core_bytes;
};

ConvPlan plan_conv(const ConvGeom &g, bool force_direct) {
  ConvPlan pl{};
  pl.M = (int64_t)g.N * g.OH * g.OW;
  pl.K = g.KH * g.KW * g.C;
  pl.Kpad = (pl.K + 15) / 16 * 16;
  pl.direct = force_direct || g.G != 1 || pl.M >= (1ll << 31) || pl.K >= (1 << 24);
  const bool pointwise = g.KH == 1 && g.KW == 1 && g.SH == 1 && g.SW == 1 && g.PT == 0 && g.PL == 0 && g.OH == g.H &&
                         g.OW == g.W && (g.C % 16) == 0;
  pl.need_im2col = !pl.direct && !pointwise;
  pl.a_bytes = pl.need_im2col ? align_up((size_t)pl.M * pl.Kpad, 256) : 0;
  pl.f_bytes = (!pl.direct && pl.Kpad != pl.K) ? align_up((size_t)g.OC * pl.Kpad, 256) : 0;
  pl.core_bytes = pl.direct ? 0 : i8_gemm_core_workspace_bytes(pl.M, g.OC);
  return pl;
}

int run_conv(GemmParams p, const int8_t *in, const int8_t *filter, const ConvGeom &g, const int32_t *filter_row_sums,
             int flags, void *workspace, size_t workspace_bytes, cudaStream_t s) {
  const int64_t outputs = (int64_t)g.N * g.OH * g.OW * g.OC;
  if (outputs == 0) return GLOWB200_OK;
  const ConvPlan pl = plan_conv(g, (flags & GLOWB200_FC_FORCE_ANY_SHAPE_KERNEL) != 0);
  if (pl.direct) {
    const int64_t blocks = (outputs + 255) / 256;
    conv2d_i8_direct_kernel<<<(unsigned)(blocks < 148 * 32 ? blocks : 148 * 32), 256, 0, s>>>(in, filter, g, p);
    GLOWB200_CUDA_OK(cudaGetLastError());
    return GLOWB200_OK;
  }
  const size_t need = pl.a_bytes + pl.f_bytes + pl.core_bytes;
  if (workspace == nullptr || workspace_bytes < need)
    return set_error(GLOWB200_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
  GLOWB200_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "workspace must be 256-byte aligned");
  uint8_t *ws = reinterpret_cast<uint8_t *>(workspace);
#if GLOWB200_CONV_SHIFTED_ROWS
  // Stride-1 windows over 64 or a multiple of 128 channels, symmetric filters: no im2col matrix.
  // The input is copied once into a padded NHWC buffer; tap (kh, kw) of output row q then is row
  // q + kh * Wp + kw of that buffer, which the contraction's loads address directly (the rows of
  // the product that fall on the padding are computed and dropped).  The scratch sized for the
  // im2col matrix is more than this needs.
  if (pl.need_im2col && g.SH == 1 && g.SW == 1 && g.DH == 1 && g.DW == 1 && (flags & GLOWB200_FC_WEIGHT_OFFSETS_ZERO) &&
      (g.C == 64 || g.C % 128 == 0) && (reinterpret_cast<uintptr_t>(in) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(filter) & 15) == 0) {
    const int Hp = g.OH + g.KH - 1, Wp = g.OW + g.KW - 1;
    // 64 channels: two neighbouring pixels per 128-byte row against a filter re-laid in tap pairs (the
    // partner of an odd last tap zero).  One tap per 64-byte k-block in the 64-byte swizzle -- no
    // wasted MMAs, a quarter fewer operand bytes, nine k-blocks instead of six for a 3 x 3 window --
    // gave the same results and a slower network (1.590 against 1.562 ms per ResNet-50 batch).
    const int pairs = (g.KW + 1) / 2;
    const int entries = g.C == 64 ? g.KH * pairs : g.KH * g.KW;
    const int64_t rows = (int64_t)g.N * Hp * Wp;
    const size_t xp_bytes = align_up((size_t)rows * g.C + 256, 256);
    const size_t fb_bytes = g.C == 64 ? align_up((size_t)g.OC * entries * 128, 256) : 0;
    if (entries <= 32 && Hp >= g.H + g.PT && Wp >= g.W + g.PL && rows < (1ll << 31) &&
        xp_bytes + fb_bytes <= pl.a_bytes + pl.f_bytes) {
      int8_t *xp = reinterpret_cast<int8_t *>(ws);
      const uint32_t b = (uint8_t)p.a_offset;
      const int64_t chunks = rows * (g.C >> 4), blocks = (chunks + 255) / 256;
      GLOWB200_CUDA_OK(launch_pdl(pad_nhwc_i8_kernel, (unsigned)(blocks < 148 * 64 ? blocks : 148 * 64), 256, 0, s, in, xp, g, Hp, Wp,
                                  (int)(b | (b << 8) | (b << 16) | (b << 24))));
      GLOWB200_CUDA_OK(cudaGetLastError());
      GLOWB200_CUDA_OK(cudaMemsetAsync(xp + rows * g.C, 0, 256, s));  // the window of the last rows reads past them
      const int8_t *bmat = filter;
      p.K = g.KH * g.KW * g.C;
      if (g.C == 64) {
        int8_t *fb = reinterpret_cast<int8_t *>(ws + xp_bytes);
        const int64_t fblocks = ((int64_t)g.OC * entries * 128 + 255) / 256;
        GLOWB200_CUDA_OK(launch_pdl(pair_taps_c64_kernel, (unsigned)(fblocks < 148 * 16 ? fblocks : 148 * 16), 256, 0, s, filter, fb, g.OC,
                                    g.KH, g.KW));
        GLOWB200_CUDA_OK(cudaGetLastError());
        bmat = fb;
        p.K = entries * 128;
      }
      p.k_corr = pl.K;
      p.N = g.OC;
      p.conv_entries = entries;
      p.conv_cpb = g.C == 64 ? 1 : g.C / 128;
      for (int e = 0; e < entries; e++)
        p.conv_row_off[e] = g.C == 64 ? (e / pairs) * Wp + 2 * (e % pairs) : (e / g.KW) * Wp + (e % g.KW);
      p.conv_hpwp = Hp * Wp;
      p.conv_wp = Wp;
      p.conv_oh = g.OH;
      p.conv_ow = g.OW;
      const int32_t *sums = filter_row_sums;
      if (sums == nullptr) {  // zeros added by the pairing do not change the sums
        int32_t *bs = reinterpret_cast<int32_t *>(ws + pl.a_bytes + pl.f_bytes);
        if (int rc = glowb200_i8_row_sums(bmat, g.OC, p.K, bs, reinterpret_cast<glowb200_stream_t>(s))) return rc;
        sums = bs;
      }
      return run_gemm_shifted_rows(p, xp, rows, g.C, bmat, sums, s);
    }
  }
#endif
  // Stride-2 windows over a multiple of 128 channels, symmetric filters: the shifted-rows form over
  // four parity planes of the padded input (see pad_parity_nhwc_i8_kernel) instead of an im2col matrix.
  if (pl.need_im2col && g.SH == 2 && g.SW == 2 && g.DH == 1 && g.DW == 1 && (g.KH > 1 || g.KW > 1) &&
      (flags & GLOWB200_FC_WEIGHT_OFFSETS_ZERO) && g.C % 128 == 0 && g.KH * g.KW <= 32 &&
      (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(filter) & 15) == 0) {
    const int Hq = g.OH + (g.KH - 1) / 2, Wq = g.OW + (g.KW - 1) / 2;
    const int64_t rows = (int64_t)g.N * Hq * Wq;  // per plane
    const size_t xp_bytes = align_up((size_t)(4 * rows) * g.C + 256, 256);
    if (4 * rows < (1ll << 31) && xp_bytes <= pl.a_bytes + pl.f_bytes) {
      int8_t *xp = reinterpret_cast<int8_t *>(ws);
      const uint32_t b = (uint8_t)p.a_offset;
      const int64_t chunks = 4 * rows * (g.C >> 4), blocks = (chunks + 255) / 256;
      GLOWB200_CUDA_OK(launch_pdl(pad_parity_nhwc_i8_kernel, (unsigned)(blocks < 148 * 64 ? blocks : 148 * 64), 256, 0, s, in, xp, g, Hq,
                                  Wq, (int)(b | (b << 8) | (b << 16) | (b << 24))));
      GLOWB200_CUDA_OK(cudaGetLastError());
      p.K = g.KH * g.KW * g.C;
      p.k_corr = pl.K;
      p.N = g.OC;
      p.conv_entries = g.KH * g.KW;
      p.conv_cpb = g.C / 128;
      for (int e = 0; e < p.conv_entries; e++) {
        const int kh = e / g.KW, kw = e % g.KW;
        p.conv_row_off[e] = (int)(((kh & 1) * 2 + (kw & 1)) * rows) + (kh >> 1) * Wq + (kw >> 1);
      }
      p.conv_hpwp = Hq * Wq;
      p.conv_wp = Wq;
      p.conv_oh = g.OH;
      p.conv_ow = g.OW;
      const int32_t *sums = filter_row_sums;
      if (sums == nullptr) {
        int32_t *bs = reinterpret_cast<int32_t *>(ws + pl.a_bytes + pl.f_bytes);
        if (int rc = glowb200_i8_row_sums(filter, g.OC, p.K, bs, reinterpret_cast<glowb200_stream_t>(s))) return rc;
        sums = bs;
      }
      return run_gemm_shifted_rows(p, xp, rows, g.C, filter, sums, s, 4 * rows);
    }
  }
  // Stride-2 windows over few channels with symmetric filters (the 7 x 7 stem over 3 channels): row
  // windows instead of an im2col matrix (see row_windows_i8_kernel).
  if (pl.need_im2col && g.SH == 2 && g.SW == 2 && g.DH == 1 && g.DW == 1 && (flags & GLOWB200_FC_WEIGHT_OFFSETS_ZERO) &&
      g.KW * g.C <= 32 && g.KH <= 8 && (reinterpret_cast<uintptr_t>(filter) & 15) == 0) {
    const int Y = g.OH + 3;
    const int64_t rows = (int64_t)g.N * Y * g.OW;
    const int64_t plane_bytes = rows * 32;
    const size_t wp_bytes = align_up((size_t)(2 * plane_bytes + (3 * (int64_t)g.OW + 1) * 32), 256);
    const size_t fb_bytes = align_up((size_t)g.OC * 256, 256);
    if (rows < (1ll << 31) && wp_bytes + fb_bytes <= pl.a_bytes + pl.f_bytes) {
      int8_t *planes = reinterpret_cast<int8_t *>(ws);
      int8_t *fb = reinterpret_cast<int8_t *>(ws + wp_bytes);
      const int64_t blocks = (2 * rows + 255) / 256;
      GLOWB200_CUDA_OK(launch_pdl(row_windows_i8_kernel, (unsigned)(blocks < 148 * 64 ? blocks : 148 * 64), 256, 0, s, in, planes, g, Y,
                                  plane_bytes, (int8_t)p.a_offset));
      GLOWB200_CUDA_OK(cudaGetLastError());
      // the four windows of the last rows reach past the second plane
      GLOWB200_CUDA_OK(cudaMemsetAsync(planes + 2 * plane_bytes, 0, wp_bytes - 2 * plane_bytes, s));
      GLOWB200_CUDA_OK(launch_pdl(window_filter_i8_kernel, (unsigned)((g.OC * 256 + 255) / 256), 256, 0, s, filter, fb, g.OC, g.KH, g.KW,
                                  g.C));
      GLOWB200_CUDA_OK(cudaGetLastError());
      int32_t *bs = reinterpret_cast<int32_t *>(ws + pl.a_bytes + pl.f_bytes);  // zeros do not change the sums, but one path
      if (int rc = glowb200_i8_row_sums(fb, g.OC, 256, bs, reinterpret_cast<glowb200_stream_t>(s))) return rc;
      p.K = 256;
      p.k_corr = pl.K;
      p.N = g.OC;
      p.conv_hpwp = Y * g.OW;
      p.conv_wp = g.OW;
      p.conv_oh = g.OH;
      p.conv_ow = g.OW;
      return run_gemm_row_windows(p, planes, rows, g.OW, fb, bs, s);
    }
  }
  const int8_t *a = in;
  if (pl.need_im2col) {
    int8_t *abuf = reinterpret_cast<int8_t *>(ws);
    const int8_t pad = (int8_t)p.a_offset;
    if ((g.C % 16) == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0) {
      const int64_t chunks = pl.M * (pl.Kpad >> 4);
      const int64_t blocks = (chunks + 255) / 256;
      const uint32_t b = (uint8_t)pad;
      GLOWB200_CUDA_OK(launch_pdl(im2col_i8_vec_kernel, (unsigned)(blocks < 148 * 64 ? blocks : 148 * 64), 256, 0, s, in, abuf, g, pl.Kpad,
                                  (int)(b | (b << 8) | (b << 16) | (b << 24))));
    } else if ((int64_t)g.KH * rows_pitch(g) <= 48 * 1024 && (int64_t)g.N * g.OH < (1ll << 31) && (pl.Kpad >> 4) <= 256 &&
               (reinterpret_cast<uintptr_t>(abuf) & 15) == 0) {
      // the KH input rows of an output image row, with their padding, fit the default shared-memory window
      const int pitch = (int)rows_pitch(g);
      im2col_i8_rows_kernel<<<(unsigned)(g.N * g.OH), 256, (size_t)g.KH * pitch, s>>>(in, abuf, g, pl.K, pl.Kpad, pad, pitch);
    } else {
      const int64_t blocks = (pl.M * pl.Kpad + 255) / 256;
      im2col_i8_kernel<<<(unsigned)(blocks < 148 * 64 ? blocks : 148 * 64), 256, 0, s>>>(in, abuf, g, pl.K, pl.Kpad, pad);
    }
    GLOWB200_CUDA_OK(cudaGetLastError());
    a = abuf;
  }
  const int8_t *b = filter;
  if (pl.f_bytes) {
    int8_t *fbuf = reinterpret_cast<int8_t *>(ws + pl.a_bytes);
    const int64_t blocks = ((int64_t)g.OC * pl.Kpad + 255) / 256;
    pad_rows_i8_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, s>>>(filter, fbuf, g.OC, pl.K, pl.Kpad);
    GLOWB200_CUDA_OK(cudaGetLastError());
    b = fbuf;
    filter_row_sums = nullptr;  // recomputed over the padded copy (same values; keeps one code path)
  }
  p.M = (int)pl.M;
  p.N = g.OC;
  p.K = pl.Kpad;
  p.k_corr = pl.K;
  return run_gemm(p, a, b, filter_row_sums, (flags & GLOWB200_FC_WEIGHT_OFFSETS_ZERO) != 0, 0, ws + pl.a_bytes + pl.f_bytes,
                  pl.core_bytes, s);
}

}  // namespace
}  // namespace glowb200

using namespace glowb200;

extern "C" size_t glowb200_conv2d_workspace_bytes(const int64_t *out_dims, const int64_t *in_dims,
                                                  const int64_t *filter_dims, const int64_t *kernels,
                                                  const int64_t *strides, const int64_t *pads, int64_t group,
                                                  const int64_t *dilation) {
  ConvGeom g;
  if (geom_from_dims(g, out_dims, in_dims, filter_dims, kernels, strides, pads, group, dilation) != GLOWB200_OK) return 0;
  const ConvPlan pl = plan_conv(g, false);
  return pl.a_bytes + pl.f_bytes + pl.core_bytes;
}

extern "C" int glowb200_channelwise_quantized_conv2d_i8_i32(
    int8_t *out, const int8_t *in, const int8_t *filter, const int32_t *bias, const int64_t *out_dims,
    const int64_t *in_dims, const int64_t *filter_dims, const int64_t *kernels, const int64_t *strides,
    const int64_t *pads, int64_t group, const int64_t *dilation, int32_t out_offset, int32_t in_offset,
    const int32_t *filter_offsets, const int32_t *bias_offsets, const int32_t *bias_pre, const int32_t *bias_post,
    const int32_t *bias_scale, const int32_t *out_pre, const int32_t *out_post, const int32_t *out_scale, int32_t act_type,
    const int32_t *act_args, const int32_t *filter_row_sums, int flags, void *workspace, size_t workspace_bytes,
    int32_t *status, glowb200_stream_t stream) {
  ConvGeom g;
  if (int rc = geom_from_dims(g, out_dims, in_dims, filter_dims, kernels, strides, pads, group, dilation)) return rc;
  if ((int64_t)g.N * g.OH * g.OW * g.OC == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(out && in && filter && bias && filter_offsets && bias_offsets && bias_pre && bias_post && bias_scale &&
                       out_pre && out_post && out_scale, "NULL tensor pointer");
  GLOWB200_REQUIRE(act_type >= 0 && act_type <= 5 && act_type != 3 && act_type != 4,
                   "fused activation %d is not defined for quantized convolution", act_type);
  GLOWB200_REQUIRE(act_type == 0 || act_type == 1 || act_args != nullptr, "activation arguments missing");
  GemmParams p{};
  p.out = out;
  p.bias = bias;
  p.b_offsets = filter_offsets;
  p.bias_offsets = bias_offsets;
  p.bias_pre = bias_pre; p.bias_post = bias_post; p.bias_scale = bias_scale;
  p.out_pre = out_pre; p.out_post = out_post; p.out_scale = out_scale;
  p.status = status;
  p.a_offset = in_offset; p.out_offset = out_offset;
  p.act_type = act_type;
  p.bias_is_i8 = (flags & GLOWB200_FC_BIAS_INT8) ? 1 : 0;
  if (act_type == 2) { p.act_args[0] = act_args[0]; p.act_args[1] = act_args[1]; }
  if (act_type == 5) { p.act_args[0] = act_args[0]; p.act_args[1] = act_args[1]; p.act_args[2] = act_args[2]; }
  return run_conv(p, in, filter, g, filter_row_sums, flags, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int glowb200_conv2d_i8_i32(
    int8_t *out, const int8_t *in, const int8_t *filter, const int32_t *bias, const int64_t *out_dims,
    const int64_t *in_dims, const int64_t *filter_dims, const int64_t *kernels, const int64_t *strides,
    const int64_t *pads, int64_t group, int32_t out_offset, int32_t in_offset, int32_t filter_offset, int32_t bias_offset,
    int32_t bias_pre, int32_t bias_post, int32_t bias_scale, int32_t out_pre, int32_t out_post, int32_t out_scale,
    const int64_t *dilation, int32_t act_type, const int32_t *act_args, int flags, void *workspace, size_t workspace_bytes,
    int32_t *status, glowb200_stream_t stream) {
  ConvGeom g;
  if (int rc = geom_from_dims(g, out_dims, in_dims, filter_dims, kernels, strides, pads, group, dilation)) return rc;
  if ((int64_t)g.N * g.OH * g.OW * g.OC == 0) return GLOWB200_OK;
  GLOWB200_REQUIRE(out && in && filter && bias, "NULL tensor pointer");
  GLOWB200_REQUIRE(act_type >= 0 && act_type <= 5 && act_type != 3 && act_type != 4,
                   "fused activation %d is not defined for quantized convolution", act_type);
  GLOWB200_REQUIRE(act_type == 0 || act_type == 1 || act_args != nullptr, "activation arguments missing");
  GemmParams p{};
  p.out = out;
  p.bias = bias;
  p.status = status;
  p.a_offset = in_offset; p.out_offset = out_offset; p.bias_offset = bias_offset;
  p.uniform = 1;
  p.u_b_offset = filter_offset;
  p.u_bias_pre = bias_pre; p.u_bias_post = bias_post; p.u_bias_scale = bias_scale;
  p.u_out_pre = out_pre; p.u_out_post = out_post; p.u_out_scale = out_scale;
  p.act_type = act_type;
  p.bias_is_i8 = (flags & GLOWB200_FC_BIAS_INT8) ? 1 : 0;
  if (act_type == 2) { p.act_args[0] = act_args[0]; p.act_args[1] = act_args[1]; }
  if (act_type == 5) { p.act_args[0] = act_args[0]; p.act_args[1] = act_args[1]; p.act_args[2] = act_args[2]; }
  if (filter_offset == 0) flags |= GLOWB200_FC_WEIGHT_OFFSETS_ZERO;
  return run_conv(p, in, filter, g, nullptr, flags, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}
