// Integer-code packing, unpacking and fused unpack+dequantize for 2/3/4/8-bit
// codes in three storage formats.  All kernels are bound by HBM traffic: every
// thread moves 16-byte vectors where the row length allows it, rows are walked
// by a grid-stride loop and the grid is sized from the SM count.
#include "common.cuh"

namespace {

__host__ __device__ constexpr int codes_per_word(int bits, int fmt) {
  // Number of codes held by one 32-bit word of packed output.
  if (fmt == DGQ_FMT_INT32_LE) return 32 / bits;
  if (bits == 4) return 8;
  if (bits == 2 && fmt == DGQ_FMT_BYTES_HI_FIRST) return 16;
  return 4;  // one code per byte
}

// Packs the codes c[0..n) (n <= codes_per_word, missing codes read as 0) into a word.
template <int BITS, int FMT>
__device__ __forceinline__ uint32_t pack_word(const uint8_t* c, int n) {
  constexpr int PER = (FMT == DGQ_FMT_INT32_LE) ? 32 / BITS
                     : (BITS == 4)              ? 8
                     : (BITS == 2 && FMT == DGQ_FMT_BYTES_HI_FIRST) ? 16 : 4;
  uint32_t w = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    uint32_t v = j < n ? c[j] : 0u;
    int sh;
    if (FMT == DGQ_FMT_INT32_LE) {
      sh = j * BITS;
    } else if (BITS == 4) {
      // byte j/2; format 1 puts the even code in the high nibble, format 2 in the low
      sh = (j >> 1) * 8 + (((j & 1) == 0) == (FMT == DGQ_FMT_BYTES_HI_FIRST) ? 4 : 0);
    } else if (BITS == 2 && FMT == DGQ_FMT_BYTES_HI_FIRST) {
      sh = (j >> 2) * 8 + (3 - (j & 3)) * 2;
    } else {
      sh = j * 8;
    }
    w |= v << sh;
  }
  return w;
}

template <int BITS, int FMT>
__device__ __forceinline__ void unpack_word(uint32_t w, uint8_t* c) {
  constexpr int PER = (FMT == DGQ_FMT_INT32_LE) ? 32 / BITS
                     : (BITS == 4)              ? 8
                     : (BITS == 2 && FMT == DGQ_FMT_BYTES_HI_FIRST) ? 16 : 4;
  constexpr bool BYTEWISE = !(FMT == DGQ_FMT_INT32_LE || BITS == 4 ||
                              (BITS == 2 && FMT == DGQ_FMT_BYTES_HI_FIRST));
  constexpr uint32_t MASK = BYTEWISE ? 0xFFu : ((1u << BITS) - 1u);
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    int sh;
    if (FMT == DGQ_FMT_INT32_LE) {
      sh = j * BITS;
    } else if (BITS == 4) {
      sh = (j >> 1) * 8 + (((j & 1) == 0) == (FMT == DGQ_FMT_BYTES_HI_FIRST) ? 4 : 0);
    } else if (BITS == 2 && FMT == DGQ_FMT_BYTES_HI_FIRST) {
      sh = (j >> 2) * 8 + (3 - (j & 3)) * 2;
    } else {
      sh = j * 8;
    }
    c[j] = (uint8_t)((w >> sh) & MASK);
  }
}

// ---- pack -------------------------------------------------------------------
// Vector path: a thread emits VW consecutive words of one row from PER*VW codes.
// Requires every row to hold a whole number of such vectors and 16-byte aligned
// rows on both sides (checked on the host).
template <int BITS, int FMT, int VW>
__global__ void __launch_bounds__(256)
pack_vec_kernel(const uint8_t* __restrict__ codes, uint32_t* __restrict__ out,
                int64_t n_vec /* rows * vec_per_row */) {
  constexpr int PER = (FMT == DGQ_FMT_INT32_LE) ? 32 / BITS
                     : (BITS == 4)              ? 8
                     : (BITS == 2 && FMT == DGQ_FMT_BYTES_HI_FIRST) ? 16 : 4;
  constexpr int NB = PER * VW;  // input bytes per thread (multiple of 8 by construction)
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec;
       v += (int64_t)gridDim.x * blockDim.x) {
    alignas(16) uint8_t c[NB];
    const uint8_t* src = codes + v * NB;
    if (NB % 16 == 0) {
#pragma unroll
      for (int i = 0; i < NB / 16; ++i)
        reinterpret_cast<uint4*>(c)[i] = __ldg(reinterpret_cast<const uint4*>(src) + i);
    } else {
#pragma unroll
      for (int i = 0; i < NB / 8; ++i)
        reinterpret_cast<uint2*>(c)[i] = __ldg(reinterpret_cast<const uint2*>(src) + i);
    }
    uint32_t w[VW];
#pragma unroll
    for (int i = 0; i < VW; ++i) w[i] = pack_word<BITS, FMT>(c + i * PER, PER);
    if (VW == 4) {
      reinterpret_cast<uint4*>(out)[v] = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
#pragma unroll
      for (int i = 0; i < VW; ++i) out[v * VW + i] = w[i];
    }
  }
}

// Generic path: one thread per output byte (byte formats) or word (format 3),
// any column count, no alignment assumptions.
template <int BITS, int FMT>
__global__ void __launch_bounds__(256)
pack_generic_kernel(const uint8_t* __restrict__ codes, uint8_t* __restrict__ out, int rows,
                    int cols, int64_t row_bytes) {
  constexpr bool WORDS = (FMT == DGQ_FMT_INT32_LE);
  constexpr int PER = codes_per_word(BITS, FMT);
  constexpr int PER_UNIT = WORDS ? PER : PER / 4;  // codes per output unit
  const int64_t units_per_row = WORDS ? row_bytes / 4 : row_bytes;
  const int64_t total = (int64_t)rows * units_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / units_per_row;
    int64_t u = i - r * units_per_row;
    int64_t c0 = u * PER_UNIT;
    int n = (int)min((int64_t)PER_UNIT, (int64_t)cols - c0);
    uint8_t c[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) c[j] = (j < n) ? codes[r * cols + c0 + j] : 0;
    uint32_t w = pack_word<BITS, FMT>(c, n);
    if (WORDS)
      reinterpret_cast<uint32_t*>(out)[i] = w;
    else
      out[i] = (uint8_t)(w & 0xFF);
  }
}

template <int BITS, int FMT>
__global__ void __launch_bounds__(256)
unpack_generic_kernel(const uint8_t* __restrict__ packed, uint8_t* __restrict__ codes, int rows,
                      int cols, int64_t row_bytes) {
  constexpr bool WORDS = (FMT == DGQ_FMT_INT32_LE);
  constexpr int PER = codes_per_word(BITS, FMT);
  constexpr int PER_UNIT = WORDS ? PER : PER / 4;
  const int64_t units_per_row = WORDS ? row_bytes / 4 : row_bytes;
  const int64_t total = (int64_t)rows * units_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / units_per_row;
    int64_t u = i - r * units_per_row;
    int64_t c0 = u * PER_UNIT;
    uint32_t w = WORDS ? reinterpret_cast<const uint32_t*>(packed)[i] : (uint32_t)packed[i];
    uint8_t c[PER];
    unpack_word<BITS, FMT>(w, c);
    int n = (int)min((int64_t)PER_UNIT, (int64_t)cols - c0);
#pragma unroll
    for (int j = 0; j < PER_UNIT; ++j)
      if (j < n) codes[r * cols + c0 + j] = c[j];
  }
}

// Vector unpack: a thread turns VW words into PER*VW code bytes.
template <int BITS, int FMT, int VW>
__global__ void __launch_bounds__(256)
unpack_vec_kernel(const uint32_t* __restrict__ packed, uint8_t* __restrict__ codes, int64_t n_vec) {
  constexpr int PER = codes_per_word(BITS, FMT);
  constexpr int NB = PER * VW;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec;
       v += (int64_t)gridDim.x * blockDim.x) {
    uint32_t w[VW];
    if (VW == 4) {
      uint4 t = __ldg(reinterpret_cast<const uint4*>(packed) + v);
      w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
    } else {
#pragma unroll
      for (int i = 0; i < VW; ++i) w[i] = __ldg(packed + v * VW + i);
    }
    alignas(16) uint8_t c[NB];
#pragma unroll
    for (int i = 0; i < VW; ++i) unpack_word<BITS, FMT>(w[i], c + i * PER);
    uint8_t* dst = codes + v * NB;
    if (NB % 16 == 0) {
#pragma unroll
      for (int i = 0; i < NB / 16; ++i)
        reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(c)[i];
    } else {
#pragma unroll
      for (int i = 0; i < NB / 8; ++i)
        reinterpret_cast<uint2*>(dst)[i] = reinterpret_cast<const uint2*>(c)[i];
    }
  }
}

// ---- unpack + dequantize ------------------------------------------------------
// One thread produces 8 consecutive outputs of one row (32 bytes of fp32 or 16 of
// bf16/fp16).  A tile of 8 columns starts at a multiple of 8, so for every format
// the packed source is a whole number of bytes at an offset computable per tile.
template <int BITS, int FMT>
__device__ __forceinline__ void load_codes8(const uint8_t* __restrict__ row, int64_t c0, int cols,
                                            uint8_t* c /*[8]*/) {
  if (FMT == DGQ_FMT_INT32_LE) {
    constexpr int PER = 32 / BITS;
    const uint32_t* wrow = reinterpret_cast<const uint32_t*>(row);
    if (PER % 8 == 0 || PER == 4) {
      // 2-bit: 16 per word, 4-bit: 8 per word, 8-bit: 4 per word -> tile inside <= 2 words
      if (PER == 4) {
        uint32_t w0 = wrow[c0 / 4];
        uint32_t w1 = (c0 + 4 < cols) ? wrow[c0 / 4 + 1] : 0u;
#pragma unroll
        for (int j = 0; j < 4; ++j) { c[j] = (w0 >> (8 * j)) & 0xFF; c[4 + j] = (w1 >> (8 * j)) & 0xFF; }
      } else {
        uint32_t w = wrow[c0 / PER];
        int base = (int)(c0 % PER) * BITS;
#pragma unroll
        for (int j = 0; j < 8; ++j) c[j] = (w >> (base + j * BITS)) & ((1u << BITS) - 1u);
      }
    } else {
      // 3-bit, 10 per word: codes of a tile may straddle words
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        int64_t cc = c0 + j;
        uint32_t w = (cc < cols) ? wrow[cc / PER] : 0u;
        c[j] = (w >> ((int)(cc % PER) * BITS)) & ((1u << BITS) - 1u);
      }
    }
  } else if (BITS == 4) {
    // 4 bytes hold the tile; the last tile of an odd-length row may be short
    int64_t b0 = c0 >> 1;
    int nb = (int)min((int64_t)4, ((int64_t)cols + 1) / 2 - b0);
    uint32_t w = 0;
    if (nb == 4 && ((reinterpret_cast<uintptr_t>(row + b0) & 3) == 0)) {
      w = *reinterpret_cast<const uint32_t*>(row + b0);
    } else {
      for (int j = 0; j < nb; ++j) w |= (uint32_t)row[b0 + j] << (8 * j);
    }
    unpack_word<4, FMT>(w, c);
  } else if (BITS == 2 && FMT == DGQ_FMT_BYTES_HI_FIRST) {
    uint32_t w = (uint32_t)row[c0 >> 2] | ((c0 + 4 < cols) ? (uint32_t)row[(c0 >> 2) + 1] << 8 : 0u);
    uint8_t t[16];
    unpack_word<2, DGQ_FMT_BYTES_HI_FIRST>(w, t);
#pragma unroll
    for (int j = 0; j < 8; ++j) c[j] = t[j];
  } else {
    if (c0 + 8 <= cols && ((reinterpret_cast<uintptr_t>(row + c0) & 7) == 0)) {
      *reinterpret_cast<uint2*>(c) = *reinterpret_cast<const uint2*>(row + c0);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] = (c0 + j < cols) ? row[c0 + j] : 0;
    }
  }
}

template <int BITS, int FMT, typename PT, typename OT>
__global__ void __launch_bounds__(256)
unpack_dequant_kernel(const uint8_t* __restrict__ packed, const PT* __restrict__ scales,
                      const PT* __restrict__ zeros, const int32_t* __restrict__ g_idx,
                      OT* __restrict__ out, int rows, int cols, int n_groups, int group_size,
                      int64_t row_bytes) {
  const int64_t tiles_per_row = ((int64_t)cols + 7) / 8;
  const int64_t total = (int64_t)rows * tiles_per_row;
  const bool vec_ok = (cols % 8 == 0);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / tiles_per_row;
    int64_t c0 = (i - r * tiles_per_row) * 8;
    uint8_t c[8];
    load_codes8<BITS, FMT>(packed + r * row_bytes, c0, cols, c);
    float v[8];
    const PT* srow = scales + r * n_groups;
    const PT* zrow = zeros + r * n_groups;
    if (g_idx == nullptr && (group_size % 8 == 0 || n_groups == 1)) {
      int g = n_groups == 1 ? 0 : (int)(c0 / group_size);
      float s = dgq_to_float<PT>(srow[g]), z = dgq_to_float<PT>(zrow[g]);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = dgq_dequant_level((float)c[j], s, z);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        int64_t cc = min(c0 + j, (int64_t)cols - 1);
        int g = g_idx ? g_idx[cc] : (n_groups == 1 ? 0 : (int)(cc / group_size));
        v[j] = dgq_dequant_level((float)c[j], dgq_to_float<PT>(srow[g]), dgq_to_float<PT>(zrow[g]));
      }
    }
    OT* dst = out + r * (int64_t)cols + c0;
    if (vec_ok) {
      if (sizeof(OT) == 4) {
        reinterpret_cast<float4*>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
      } else {
        alignas(16) OT t[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = dgq_from_float<OT>(v[j]);
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(t);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (c0 + j < cols) dst[j] = dgq_from_float<OT>(v[j]);
    }
  }
}

// Wide path for the layout the quantized layers store (4-bit, two codes per byte, low
// nibble first) when rows hold whole 8-column words and groups are multiples of 8 columns.
// The matrix is walked as a flat array of 32-bit words (8 codes each).  A thread handles
// four words that are 32 words apart, so that every load instruction of a warp reads 128
// consecutive bytes and every store instruction writes 512 (bf16/fp16) or 1024 (fp32)
// consecutive bytes; the four independent loads are in flight together.  The kernel has to
// stay below about 60 instructions per word to remain bound by HBM, so the row and column of
// a word come from one 32-bit division per thread and step (the other three words follow by
// addition), the group from a shift when the group size is a power of two, and the codes
// become floats by the 2^23 trick on the FMA pipe instead of the conversion unit.
template <typename PT, typename OT>
__global__ void __launch_bounds__(256)
unpack_dequant_wide4_kernel(const uint32_t* __restrict__ packed, const PT* __restrict__ scales,
                            const PT* __restrict__ zeros, OT* __restrict__ out, uint32_t n_words,
                            uint32_t words_per_row, int n_groups, uint32_t group_words,
                            int group_shift) {
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t n_warps = (gridDim.x * blockDim.x) >> 5;
  for (uint64_t base64 = (uint64_t)warp_global * 128; base64 < n_words; base64 += (uint64_t)n_warps * 128) {
    const uint32_t base = (uint32_t)base64;
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t wi = base + q * 32 + lane;
      w[q] = wi < n_words ? __ldg(packed + wi) : 0u;
    }
    uint32_t r = (base + lane) / words_per_row;
    uint32_t c = (base + lane) - r * words_per_row;     // word within the row
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t wi = base + q * 32 + lane;
      if (wi >= n_words) break;
      const uint32_t g = n_groups == 1 ? 0u : (group_shift >= 0 ? c >> group_shift : c / group_words);
      const float s = dgq_to_float<PT>(scales[(uint64_t)r * n_groups + g]);
      const float z = dgq_to_float<PT>(zeros[(uint64_t)r * n_groups + g]);
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float code = __uint_as_float(0x4B000000u | ((w[q] >> (4 * j)) & 0xFu)) - 8388608.f;
        v[j] = dgq_dequant_level(code, s, z);
      }
      OT* dst = out + (uint64_t)wi * 8;
      if (sizeof(OT) == 4) {
        reinterpret_cast<float4*>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
      } else {
        alignas(16) OT t[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = dgq_from_float<OT>(v[j]);
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(t);
      }
      c += 32;
      while (c >= words_per_row) { c -= words_per_row; ++r; }
    }
  }
}

bool valid_bits(int b) { return b == 2 || b == 3 || b == 4 || b == 8; }
bool valid_fmt(int f) { return f >= 1 && f <= 3; }

#define DGQ_DISPATCH_BITS_FMT(bits, fmt, CALL)                          \
  switch ((bits) * 10 + (fmt)) {                                        \
    case 21: { CALL(2, 1); } break; case 22: { CALL(2, 2); } break;     \
    case 23: { CALL(2, 3); } break; case 31: { CALL(3, 1); } break;     \
    case 32: { CALL(3, 2); } break; case 33: { CALL(3, 3); } break;     \
    case 41: { CALL(4, 1); } break; case 42: { CALL(4, 2); } break;     \
    case 43: { CALL(4, 3); } break; case 81: { CALL(8, 1); } break;     \
    case 82: { CALL(8, 2); } break; case 83: { CALL(8, 3); } break;     \
    default: return DGQ_ERR_ARG;                                        \
  }

}  // namespace

DGQ_EXPORT int64_t dgq_packed_row_bytes(int32_t cols, int32_t bits, int32_t format) {
  if (cols <= 0 || !valid_bits(bits) || !valid_fmt(format)) return DGQ_ERR_ARG;
  if (format == DGQ_FMT_INT32_LE) return 4 * dgq_cdiv(cols, 32 / bits);
  if (format == DGQ_FMT_BYTES_HI_FIRST) {
    if (bits == 4) return cols % 2 ? DGQ_ERR_ARG : cols / 2;
    if (bits == 2) return cols % 4 ? DGQ_ERR_ARG : cols / 4;
    return cols;
  }
  return bits == 4 ? (cols + 1) / 2 : cols;
}

DGQ_EXPORT int32_t dgq_pack(const uint8_t* codes, int32_t rows, int32_t cols, int32_t bits,
                            int32_t format, void* packed, void* stream) {
  DGQ_REQUIRE(codes && packed && rows > 0 && cols > 0, DGQ_ERR_ARG);
  int64_t row_bytes = dgq_packed_row_bytes(cols, bits, format);
  DGQ_REQUIRE(row_bytes > 0, DGQ_ERR_ARG);
  cudaStream_t st = dgq_stream(stream);
  const int per = codes_per_word(bits, format);
  // vector path: 4 words (16 bytes) per thread when rows are whole vectors and aligned
  const int vw = 4;
  const bool vec = (cols % (per * vw) == 0) && dgq_aligned(codes, 16) && dgq_aligned(packed, 16) &&
                   ((per * vw) % 8 == 0);
  if (vec) {
    int64_t n_vec = (int64_t)rows * (cols / (per * vw));
    unsigned grid = dgq_grid(n_vec, 256);
#define CALL(B, F) \
  pack_vec_kernel<B, F, 4><<<grid, 256, 0, st>>>(codes, reinterpret_cast<uint32_t*>(packed), n_vec)
    DGQ_DISPATCH_BITS_FMT(bits, format, CALL)
#undef CALL
  } else {
    int64_t units = (int64_t)rows * (format == DGQ_FMT_INT32_LE ? row_bytes / 4 : row_bytes);
    unsigned grid = dgq_grid(units, 256);
#define CALL(B, F)                                                                          \
  pack_generic_kernel<B, F><<<grid, 256, 0, st>>>(codes, reinterpret_cast<uint8_t*>(packed), \
                                                  rows, cols, row_bytes)
    DGQ_DISPATCH_BITS_FMT(bits, format, CALL)
#undef CALL
  }
  return dgq_launch_status();
}

DGQ_EXPORT int32_t dgq_unpack(const void* packed, int32_t rows, int32_t cols, int32_t bits,
                              int32_t format, uint8_t* codes, void* stream) {
  DGQ_REQUIRE(codes && packed && rows > 0 && cols > 0, DGQ_ERR_ARG);
  int64_t row_bytes = dgq_packed_row_bytes(cols, bits, format);
  DGQ_REQUIRE(row_bytes > 0, DGQ_ERR_ARG);
  cudaStream_t st = dgq_stream(stream);
  const int per = codes_per_word(bits, format);
  const bool vec = (cols % (per * 4) == 0) && dgq_aligned(codes, 16) && dgq_aligned(packed, 16) &&
                   ((per * 4) % 8 == 0);
  if (vec) {
    int64_t n_vec = (int64_t)rows * (cols / (per * 4));
    unsigned grid = dgq_grid(n_vec, 256);
#define CALL(B, F) \
  unpack_vec_kernel<B, F, 4><<<grid, 256, 0, st>>>(reinterpret_cast<const uint32_t*>(packed), codes, n_vec)
    DGQ_DISPATCH_BITS_FMT(bits, format, CALL)
#undef CALL
  } else {
    int64_t units = (int64_t)rows * (format == DGQ_FMT_INT32_LE ? row_bytes / 4 : row_bytes);
    unsigned grid = dgq_grid(units, 256);
#define CALL(B, F)                                                                    \
  unpack_generic_kernel<B, F><<<grid, 256, 0, st>>>(reinterpret_cast<const uint8_t*>(packed), \
                                                    codes, rows, cols, row_bytes)
    DGQ_DISPATCH_BITS_FMT(bits, format, CALL)
#undef CALL
  }
  return dgq_launch_status();
}

namespace {
template <int B, int F, typename PT>
int32_t launch_ud_out(const void* packed, const void* scales, const void* zeros,
                      const int32_t* g_idx, int rows, int cols, int n_groups, int group_size,
                      int out_dtype, void* out, int64_t row_bytes, cudaStream_t st) {
  int64_t tiles = (int64_t)rows * dgq_cdiv(cols, 8);
  unsigned grid = dgq_grid(tiles, 256);
  const uint8_t* p = reinterpret_cast<const uint8_t*>(packed);
  const PT* s = reinterpret_cast<const PT*>(scales);
  const PT* z = reinterpret_cast<const PT*>(zeros);
  if (B == 4 && F == DGQ_FMT_BYTES_LO_FIRST && g_idx == nullptr && cols % 8 == 0 &&
      (n_groups == 1 || group_size % 8 == 0) && dgq_aligned(packed, 4) &&
      (int64_t)rows * (cols / 8) < (int64_t)1 << 31) {
    const uint32_t n_words = (uint32_t)((int64_t)rows * (cols / 8));
    const unsigned wgrid = dgq_grid(dgq_cdiv(n_words, 4), 256);
    const uint32_t* p4 = reinterpret_cast<const uint32_t*>(packed);
    const uint32_t group_words = n_groups == 1 ? (uint32_t)(cols / 8) : (uint32_t)(group_size / 8);
    int group_shift = -1;
    for (int sh = 0; sh < 31; ++sh)
      if (group_words == (1u << sh)) group_shift = sh;
    switch (out_dtype) {
      case DGQ_F32:
        unpack_dequant_wide4_kernel<PT, float><<<wgrid, 256, 0, st>>>(
            p4, s, z, reinterpret_cast<float*>(out), n_words, (uint32_t)(cols / 8), n_groups,
            group_words, group_shift);
        return dgq_launch_status();
      case DGQ_F16:
        unpack_dequant_wide4_kernel<PT, __half><<<wgrid, 256, 0, st>>>(
            p4, s, z, reinterpret_cast<__half*>(out), n_words, (uint32_t)(cols / 8), n_groups,
            group_words, group_shift);
        return dgq_launch_status();
      case DGQ_BF16:
        unpack_dequant_wide4_kernel<PT, __nv_bfloat16><<<wgrid, 256, 0, st>>>(
            p4, s, z, reinterpret_cast<__nv_bfloat16*>(out), n_words, (uint32_t)(cols / 8),
            n_groups, group_words, group_shift);
        return dgq_launch_status();
      default:
        return DGQ_ERR_ARG;
    }
  }
  switch (out_dtype) {
    case DGQ_F32:
      unpack_dequant_kernel<B, F, PT, float><<<grid, 256, 0, st>>>(
          p, s, z, g_idx, reinterpret_cast<float*>(out), rows, cols, n_groups, group_size, row_bytes);
      break;
    case DGQ_F16:
      unpack_dequant_kernel<B, F, PT, __half><<<grid, 256, 0, st>>>(
          p, s, z, g_idx, reinterpret_cast<__half*>(out), rows, cols, n_groups, group_size, row_bytes);
      break;
    case DGQ_BF16:
      unpack_dequant_kernel<B, F, PT, __nv_bfloat16><<<grid, 256, 0, st>>>(
          p, s, z, g_idx, reinterpret_cast<__nv_bfloat16*>(out), rows, cols, n_groups, group_size,
          row_bytes);
      break;
    default:
      return DGQ_ERR_ARG;
  }
  return dgq_launch_status();
}
}  // namespace

DGQ_EXPORT int32_t dgq_unpack_dequant(const void* packed, const void* scales, const void* zeros,
                                      const int32_t* g_idx, int32_t rows, int32_t cols,
                                      int32_t n_groups, int32_t bits, int32_t group_size,
                                      int32_t format, int32_t param_dtype, int32_t out_dtype,
                                      void* out, void* stream) {
  DGQ_REQUIRE(packed && scales && zeros && out && rows > 0 && cols > 0 && n_groups > 0, DGQ_ERR_ARG);
  int64_t row_bytes = dgq_packed_row_bytes(cols, bits, format);
  DGQ_REQUIRE(row_bytes > 0, DGQ_ERR_ARG);
  DGQ_REQUIRE(param_dtype == DGQ_F32 || param_dtype == DGQ_F16, DGQ_ERR_ARG);
  if (g_idx == nullptr && n_groups > 1) {
    DGQ_REQUIRE(group_size > 0 && dgq_cdiv(cols, group_size) <= n_groups, DGQ_ERR_ARG);
  }
  DGQ_REQUIRE(dgq_aligned(out, 16), DGQ_ERR_ALIGN);
  cudaStream_t st = dgq_stream(stream);
#define CALL(B, F)                                                                               \
  return param_dtype == DGQ_F32                                                                  \
             ? launch_ud_out<B, F, float>(packed, scales, zeros, g_idx, rows, cols, n_groups,    \
                                          group_size, out_dtype, out, row_bytes, st)             \
             : launch_ud_out<B, F, __half>(packed, scales, zeros, g_idx, rows, cols, n_groups,   \
                                           group_size, out_dtype, out, row_bytes, st)
  DGQ_DISPATCH_BITS_FMT(bits, format, CALL)
#undef CALL
  return DGQ_ERR_ARG;
}
