"""Numeric constants of the backend operator surface.

Values are those of the reference binding (adamah-MAIN/adamah/__init__.py:36-137)
so that code written against ``adamah`` works unchanged; ``DTYPE_GGUF_*`` are
additive extensions for maps that keep weights as native GGUF blocks.
"""
# map element types (adamah-MAIN/adamah/__init__.py DTYPE_*; adamah.c:2698-2824)
DTYPE_F32 = 0
DTYPE_BF16 = 1
DTYPE_Q8 = 2
DTYPE_Q4 = 3
DTYPE_Q6 = 4
# extensions: weights stored as GGUF blocks (18 B / 32 and 144 B / 256)
DTYPE_GGUF_Q4_0 = 16
DTYPE_GGUF_Q4_K = 17
DTYPE_GGUF_Q8_0 = 18
DTYPE_GGUF_Q5_0 = 19

# status codes (adamah.c:23-28)
ADAMAH_OK = 0
ADAMAH_ERR_BACKEND = -1
ADAMAH_ERR_MEMORY = -2
ADAMAH_ERR_INVALID = -3
ADAMAH_ERR_NOT_FOUND = -4

# unary ops (map_op1)
OP_NEG = 0; OP_ABS = 1; OP_SQRT = 2; OP_EXP = 3; OP_LOG = 4; OP_TANH = 5; OP_RELU = 6; OP_GELU = 7
OP_SIN = 8; OP_COS = 9; OP_TAN = 10; OP_ASIN = 11; OP_ACOS = 12; OP_ATAN = 13; OP_SINH = 14; OP_COSH = 15
OP_SIGMOID = 16; OP_SWISH = 17; OP_MISH = 18; OP_SELU = 19; OP_ELU = 20; OP_LEAKY_RELU = 21
OP_CEIL = 22; OP_FLOOR = 23; OP_ROUND = 24; OP_SIGN = 25; OP_RECIPROCAL = 26; OP_SQUARE = 27
OP_CUBE = 28; OP_SOFTPLUS = 29; OP_HARDSIGMOID = 30; OP_HARDSWISH = 31; OP_EXPM1 = 32; OP_LOG1P = 33
# binary ops (map_op2)
OP_ADD = 0; OP_SUB = 1; OP_MUL = 2; OP_DIV = 3; OP_POW = 4; OP_MIN = 5; OP_MAX = 6; OP_MOD = 7
OP_EQ = 8; OP_NE = 9; OP_LT = 10; OP_LE = 11; OP_GT = 12; OP_GE = 13; OP_AND = 14; OP_OR = 15; OP_XOR = 16
OP_GEGLU = 34
OP_SWIGLU = 35
# broadcast ops (map_broadcast)
BROADCAST_MUL = 0; BROADCAST_DIV = 1; BROADCAST_ADD = 2; BROADCAST_SUB = 3

# fusion scheduler modes (adamah.c:66-68)
FUSION_SCHEDULER_LEGACY = 0
FUSION_SCHEDULER_ALIAS_SAFE = 1
FUSION_SCHEDULER_LEVEL_BATCHED = 2

# decode-plan op kinds and runtime sentinels (adamah.c:72-99)
DECODE_RUNTIME_POS = 0xFFFFFFFE
DECODE_RUNTIME_SEQ_LEN = 0xFFFFFFFD
DECODE_OP_NOP = 0
DECODE_OP_FUSION_FLUSH = 1
DECODE_OP_FUSION_ENABLE = 2
DECODE_OP_OP1 = 10
DECODE_OP_OP2 = 11
DECODE_OP_RMSNORM = 12
DECODE_OP_RMSNORM_X = 13
DECODE_OP_RMSNORM_ADD = 14
DECODE_OP_ROPE = 15
DECODE_OP_MATMUL_T = 16
DECODE_OP_MATMUL_T_XQ4 = 19
DECODE_OP_QK_NORM_ROPE_X = 23
DECODE_OP_ROW_COPY_OFFSET = 24
DECODE_OP_ATTN_SOFTMAX_VALUE = 25

# ggml tensor types accepted by map_upload_gguf_blocks
GGML_TYPE_F32 = 0
GGML_TYPE_Q4_0 = 2
GGML_TYPE_Q5_0 = 6
GGML_TYPE_Q8_0 = 8
GGML_TYPE_Q4_K = 12
# map dtype that stores each block type as it is in the file
GGUF_MAP_DTYPE = {GGML_TYPE_Q4_0: DTYPE_GGUF_Q4_0, GGML_TYPE_Q4_K: DTYPE_GGUF_Q4_K, GGML_TYPE_Q8_0: DTYPE_GGUF_Q8_0, GGML_TYPE_Q5_0: DTYPE_GGUF_Q5_0}
