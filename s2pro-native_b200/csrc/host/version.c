#include "s2p_b200_ext.h"
const char* s2p_b200_version(void) { return "s2pro-b200 0.1 sm_100a"; }
