from morphocore_b200._native import ops  # noqa: F401  torch.ops.morphocore, backed by the sm_100a kernels
