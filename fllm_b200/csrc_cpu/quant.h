// Block formats of the packed weight types and their host-side codecs.
//
// Layouts are the on-disk GGUF ones (block sizes / bytes: Q4_0 32/18, Q4_1 32/20, Q5_0 32/22, Q5_1 32/24,
// Q8_0 32/34, Q2_K 256/84, Q3_K 256/110, Q4_K 256/144, Q5_K 256/176, Q6_K 256/210, IQ4_NL 32/18,
// IQ4_XS 256/136, MXFP4 32/17) plus NVFP4 (16 e2m1 values
// per e4m3 scale) and block-wise FP8 e4m3. Type ids are the GGML ones where one exists
// (cf. rust/gguf-probe/src/quant_types.rs:44-80).
#pragma once
#include <stddef.h>
#include <stdint.h>

#define FLLM_API extern "C" __attribute__((visibility("default")))

enum FllmType : int {
  FLLM_F32 = 0,
  FLLM_F16 = 1,
  FLLM_Q4_0 = 2,
  FLLM_Q4_1 = 3,
  FLLM_Q5_0 = 6,
  FLLM_Q5_1 = 7,
  FLLM_Q8_0 = 8,
  FLLM_Q2_K = 10,
  FLLM_Q3_K = 11,
  FLLM_Q4_K = 12,
  FLLM_Q5_K = 13,
  FLLM_Q6_K = 14,
  FLLM_Q8_K = 15,
  FLLM_IQ4_NL = 20,
  FLLM_IQ4_XS = 23,
  FLLM_BF16 = 30,
  FLLM_MXFP4 = 39,
  FLLM_NVFP4 = 1001,     // not a GGML id: 16 x e2m1 + 1 x ue4m3 scale = 9 bytes / 16 values
  FLLM_FP8_E4M3 = 1002,  // raw e4m3 bytes (scales are kept separately)
};

constexpr int QK_K = 256;

#pragma pack(push, 1)
struct BlockQ4_0 { uint16_t d; uint8_t qs[16]; };
struct BlockQ4_1 { uint16_t d; uint16_t m; uint8_t qs[16]; };
struct BlockQ5_0 { uint16_t d; uint8_t qh[4]; uint8_t qs[16]; };
struct BlockQ5_1 { uint16_t d; uint16_t m; uint8_t qh[4]; uint8_t qs[16]; };
struct BlockQ8_0 { uint16_t d; int8_t qs[32]; };
struct BlockQ2K { uint8_t scales[16]; uint8_t qs[64]; uint16_t d; uint16_t dmin; };
struct BlockQ3K { uint8_t hmask[32]; uint8_t qs[64]; uint8_t scales[12]; uint16_t d; };
struct BlockIQ4NL { uint16_t d; uint8_t qs[16]; };
struct BlockIQ4XS { uint16_t d; uint16_t scales_h; uint8_t scales_l[4]; uint8_t qs[128]; };
struct BlockQ4K { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qs[128]; };
struct BlockQ5K { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qh[32]; uint8_t qs[128]; };
struct BlockQ6K { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; };
struct BlockQ8K { float d; int8_t qs[256]; int16_t bsums[16]; };
struct BlockMXFP4 { uint8_t e; uint8_t qs[16]; };
struct BlockNVFP4 { uint8_t scale; uint8_t qs[8]; };
#pragma pack(pop)

static_assert(sizeof(BlockQ4K) == 144, "Q4_K block must be 144 bytes");
static_assert(sizeof(BlockQ5K) == 176, "Q5_K block must be 176 bytes");
static_assert(sizeof(BlockQ6K) == 210, "Q6_K block must be 210 bytes");
static_assert(sizeof(BlockQ4_1) == 20 && sizeof(BlockQ5_0) == 22 && sizeof(BlockQ5_1) == 24, "legacy 4/5-bit blocks");
static_assert(sizeof(BlockQ2K) == 84 && sizeof(BlockQ3K) == 110, "Q2_K / Q3_K blocks");
static_assert(sizeof(BlockIQ4NL) == 18 && sizeof(BlockIQ4XS) == 136, "IQ4 blocks");
static_assert(sizeof(BlockQ8_0) == 34 && sizeof(BlockQ4_0) == 18 && sizeof(BlockMXFP4) == 17, "legacy blocks");

float fllm_fp16_to_fp32(uint16_t h);
uint16_t fllm_fp32_to_fp16(float f);
float fllm_bf16_to_fp32(uint16_t h);
uint16_t fllm_fp32_to_bf16(float f);
float fllm_e4m3_to_fp32(uint8_t v);
uint8_t fllm_fp32_to_e4m3(float f);
float fllm_e2m1_to_fp32(uint8_t v);
uint8_t fllm_fp32_to_e2m1(float f);

// elements per block / bytes per block; 0 for unknown types
FLLM_API int fllm_block_size(int type);
FLLM_API int fllm_block_bytes(int type);
FLLM_API int64_t fllm_row_bytes(int type, int64_t ncols);
// row-wise codecs; ncols must be a multiple of the block size
FLLM_API int fllm_quantize(int type, const float* src, void* dst, int64_t nrows, int64_t ncols);
FLLM_API int fllm_dequantize(int type, const void* src, float* dst, int64_t nrows, int64_t ncols);

void quantize_row_q8_K(const float* x, BlockQ8K* y, int64_t n);
float dot_q4_K_q8_K(const BlockQ4K* w, const BlockQ8K* a, int64_t nblocks);
float dot_q6_K_q8_K(const BlockQ6K* w, const BlockQ8K* a, int64_t nblocks);
