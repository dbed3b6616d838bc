"""Hand-written sm_100a kernels (sources under ``csrc/``) and their Python bindings."""
