"""B200-native drop-in for the SparseCore hot path of jax-tpu-embedding."""
