"""Workloads and glue above the collectives: MoE routing (moe), parallelism strategies as
communication plans (strategies), training-loop hooks (hooks), the CPU ring over gloo (cpu_ring)."""
