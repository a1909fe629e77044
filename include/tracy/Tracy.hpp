// Tracy zone macros compile to nothing: the reference guards its zones with TRACY_ENABLE
// (examples/train_mlp.cpp:16-18); NVTX / CUDA events are used for profiling on B200 instead.
#pragma once
#ifndef ZoneScoped
#define ZoneScoped
#define ZoneScopedN(name)
#define ZoneNamedN(var, name, active)
#define FrameMark
#endif
