// Head dimension 64 instantiation of the flash attention backward kernels; exported as rlb_flash_attn_bwd_d64.
#define RLB_HD 64
#define RLB_NAME(x) x##_d64
#include "flash_attention_bwd.cu"
