"""Model building blocks: attention, RoPE, norms, MLPs, MoE, LM head, transformer models."""
