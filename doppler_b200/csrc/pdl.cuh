// Programmatic dependent launch (griddepcontrol) helpers.
//
// pdl_launch(): lets the next kernel in the stream start being scheduled now.
// pdl_wait():   blocks until the previous kernel in the stream has completed and its
//               writes are visible.  Both are no-ops for a kernel launched without the
//               programmatic-serialization attribute.
// Rule used throughout: a kernel calls pdl_launch() first, may then touch only data no
// earlier kernel of the step writes (the packed weights), calls pdl_wait(), and only then
// reads activations or writes anything.
#pragma once
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
