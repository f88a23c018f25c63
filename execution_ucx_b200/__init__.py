"""execution_ucx_b200: a Blackwell-native asynchronous communication runtime.

Layers (bottom to top):

* ``ops``       -- sm_100a data-plane kernels behind a C ABI (tensor send/recv with
                  pack/cast/handler fusion, MoE dispatch/combine, tcgen05 remote GEMM)
* ``parallel``  -- peer-mapped buffers and rank groups
* ``models``    -- the flagship workloads built from the ops (tensor RPC echo,
                  remote-GEMM RPC, MoE all-to-all, small-message RPC storm)
* ``axon``      -- the Python face of the native runtime (AxonRuntime, devices,
                  DLPack interop), same surface as the reference's ``axon`` package
* ``utils``     -- device timing, clock sampling, roofline arithmetic

The host runtime (sender/receiver executor, active-message context, rpc core,
axon worker, storage) is C++ under ``csrc/eux`` and is reached through
``execution_ucx_b200.axon``.
"""
__version__ = "0.2.0"
