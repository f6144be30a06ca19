"""Built-in patch patterns of the MoE decode path."""
