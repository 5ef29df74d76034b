// build_info.cu — identification string of the library.
#include "chromofold_b200/sealed_kv.h"

#define CFB_STR2(x) #x
#define CFB_STR(x) CFB_STR2(x)

extern "C" const char *cf_b200_build_info(void) {
    return "chromofold_b200 abi " CFB_STR(CF_B200_ABI_VERSION) " format " CFB_STR(CF_B200_FORMAT_VERSION)
           " sm_100a cuda " CFB_STR(__CUDACC_VER_MAJOR__) "." CFB_STR(__CUDACC_VER_MINOR__);
}
