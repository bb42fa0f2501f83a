"""B200-native drop-in for the per-batch temporal-embedding path of Orca (TGN with cached
historical embeddings)."""
