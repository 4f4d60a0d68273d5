"""Hot-path operators: autograd functions over the hand-written sm_100a kernels."""
