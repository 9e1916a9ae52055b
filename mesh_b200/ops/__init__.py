"""Python entry points over the sm_100a kernels."""
