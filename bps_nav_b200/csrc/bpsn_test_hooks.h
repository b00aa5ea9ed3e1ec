/* Exports of libbpsn.so that exist for its tests only; not part of the interface in
 * include/bpsn.h and subject to change. */
#ifndef BPSN_TEST_HOOKS_H
#define BPSN_TEST_HOOKS_H

#include "../../include/bpsn.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Diagnostic.  Scenes that are searched in global memory keep, per warp, a node array that is
 * not wiped between searches: a node counts as visited when it carries the number of the
 * running search (15 bits; when the number wraps the array is wiped once).  This call sets
 * that number for every such array of `group`, so that a test can cross the wrap after a few
 * steps instead of after 32767 searches.  No step may be in flight.  Groups whose scenes all
 * fit in shared memory have no such arrays; the call then does nothing. */
int32_t bpsn_debug_set_search_count(bpsn_sim* sim, uint32_t group, uint32_t count);

/* Diagnostic.  Large batches of fixed scenes have two forms of the step kernel (entry by entry,
 * or 32 entries searched and then finished one per lane) and choose between them step by step
 * from the number of entries the step before listed.  mode 1: always the second form where the
 * group has it, 2: never, 0: back to the choice. */
int32_t bpsn_debug_force_batched(bpsn_sim* sim, uint32_t group, int32_t mode);

#ifdef __cplusplus
}
#endif

#endif /* BPSN_TEST_HOOKS_H */
