"""Tensor-free host policy (scheduler, paging, prefix index, speculative math, samplers, constraints,
stream text segmentation). The hot pieces are C++ (libswb200_host.so) with these modules as bindings."""
