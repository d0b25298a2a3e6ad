"""Import-path shim: the reference imports its compiled kernels as
`runtime.sq_fp8_kernels` (LLMQRT/runtime_refact/nn_models/modules/linear/linear_awq.py:24-38;
extension name in LLMQRT/setup_runtime.py:20-24).  With this repository on
sys.path the unmodified reference module dispatches into the sm_100a kernels."""
