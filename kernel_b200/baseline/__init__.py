"""Library-path implementations (torch.distributed collectives + cuBLAS): the
algorithms the reference ships, kept as the measured baseline of every fused op."""
