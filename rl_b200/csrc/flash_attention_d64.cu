// Head dimension 64 instantiation of the flash attention forward kernel (Llama-3.2-1B, Qwen2.5-0.5B and other small
// models): the same source with one [rows x 64] swizzle atom per operand tile; exported as rlb_flash_attn_fwd_d64 and
// rlb_attn_delta_d64.
#define RLB_HD 64
#define RLB_NAME(x) x##_d64
#include "flash_attention.cu"
