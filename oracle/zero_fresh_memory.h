/* Forced into the one reference file that allocates host blocks (src/syncedmem.cpp) when it is
 * compiled as the parity oracle: fresh blocks read as zero.
 *
 * The reference hands out host memory without clearing it (src/syncedmem.cpp:42-46, the memset is
 * commented out), several of its layers decide whether their vector of ones needs filling by
 * looking at the vector's last element only (src/layers/bias_layer.cpp:62-65 and the same idiom in
 * the Scale, InnerProduct and Convolution bias paths), and other places count on fresh memory being
 * zero.  On pages fresh from the kernel that holds, which is the state the reference was written
 * and tested in; with recycled heap memory its results depend on what the process ran before (seen
 * here as a Bias output that was off by a stale multiplier).  An oracle must not depend on the
 * allocation history, so its fresh blocks are zeroed; together with running every oracle net in a
 * thread of its own (the reference's pool is per thread) each net starts from that state.
 * TEST INFRASTRUCTURE ONLY, like everything under oracle/. */
#ifndef ORACLE_ZERO_FRESH_MEMORY_H_
#define ORACLE_ZERO_FRESH_MEMORY_H_
#include <stdlib.h>
#define malloc(n) calloc(1, (n))
#endif
