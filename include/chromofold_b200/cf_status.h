/* cf_status.h — status codes and limits shared by every entry point of this library.
 * Values are those of the reference's include/chromofold/chromofold.h:22-30 so that a caller compiled
 * against the reference headers reads the same numbers. */
#ifndef CHROMOFOLD_B200_CF_STATUS_H
#define CHROMOFOLD_B200_CF_STATUS_H

#ifdef __cplusplus
extern "C" {
#endif

#ifndef CHROMOFOLD_H /* the reference header defines the same enum; never define it twice */
typedef enum cf_status {
    CF_OK = 0,
    CF_ERR_INVALID_ARGUMENT = 1,
    CF_ERR_UNSUPPORTED = 2,
    CF_ERR_CUDA = 3
} cf_status;

#define CF_KV_MAX_HEAD_DIM 128
#define CF_KV_MAX_WINDOW 512
#endif

#ifdef __cplusplus
}
#endif

#endif
