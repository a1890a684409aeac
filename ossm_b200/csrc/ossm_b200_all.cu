// Single translation unit of libossm_b200.so (keeps the device status word and
// the helpers in one module without relocatable device code).
#include <cstring>

#include "common.cu"
#include "lti_scan.cu"
#include "linoss_generic.cu"
#include "sdlinoss_scan.cu"
#include "selective_scan.cu"
