"""The plain, slow implementation the engine is compared with (numpy, whole sequences, no cache)."""
