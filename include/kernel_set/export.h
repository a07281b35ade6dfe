/*
 * Linkage and visibility macros for the quantized-GEMM drop-in library.
 *
 * Replaces include/kernel_set/export.h:12-29 of the reference project. The
 * library is compiled with -fvisibility=hidden, so only symbols carrying
 * KS_API are visible to a binding's dlopen/dlsym.
 */
#ifndef KERNEL_SET_EXPORT_H_
#define KERNEL_SET_EXPORT_H_

#if defined(_WIN32) || defined(__CYGWIN__)
#  if defined(KERNEL_SET_BUILD)
#    define KS_API __declspec(dllexport)
#  else
#    define KS_API __declspec(dllimport)
#  endif
#else
#  define KS_API __attribute__((visibility("default")))
#endif

#if defined(__cplusplus)
#  define KS_BEGIN_EXTERN_C extern "C" {
#  define KS_END_EXTERN_C }
#else
#  define KS_BEGIN_EXTERN_C
#  define KS_END_EXTERN_C
#endif

#endif /* KERNEL_SET_EXPORT_H_ */
