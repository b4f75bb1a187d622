"""Parallelism: tensor parallel (symmetric memory + fused NVLink kernels) and ZeRO data parallel."""
