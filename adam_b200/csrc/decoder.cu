#include "common.cuh"
namespace ab { void decoder_destroy_all() {} }
