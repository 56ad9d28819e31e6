/* s2pro-b200 — additive entry points that have no counterpart in the
 * reference's headers.  Everything the reference's callers use is in
 * s2p_b200_abi.h; a drop-in build never needs this file. */
#ifndef S2P_B200_EXT_H
#define S2P_B200_EXT_H

#include "s2p_b200_abi.h"

#ifdef __cplusplus
extern "C" {
#endif
/* the library is built with hidden visibility; only what is declared here is exported */
#pragma GCC visibility push(default)

/* Library identification: "s2pro-b200 <version> sm_100a". */
const char* s2p_b200_version(void);

#pragma GCC visibility pop
#ifdef __cplusplus
}
#endif
#endif
