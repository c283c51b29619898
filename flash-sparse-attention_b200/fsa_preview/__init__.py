"""One-step NSA decode on the sm_100a kernels (the reference's ``fsa_preview`` package)."""
