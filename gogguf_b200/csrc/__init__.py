"""CUDA sources (sm_100a), their build, and their Python face."""
