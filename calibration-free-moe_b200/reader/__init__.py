"""Sparse MoE decode reader: budgets, sketch and the CUDA operator."""
