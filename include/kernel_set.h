/* Umbrella header: everything the quantized-GEMM drop-in library exports. */
#ifndef KERNEL_SET_H_
#define KERNEL_SET_H_
#include "kernel_set/types.h"
#include "kernel_set/runtime.h"
#include "kernel_set/gemm.h"
#include "kernel_set/quant.h"
#include "kernel_set/moe.h"
#include "kernel_set/activation.h"
#include "kernel_set/norm.h"
#endif /* KERNEL_SET_H_ */
