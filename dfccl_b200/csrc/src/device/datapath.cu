// The one translation unit that holds the out-of-line reduce / copy bodies (device and host code).
#define DF_DATAPATH_IMPL
#include "datapath.h"
