"""Model stacks: decoder skeleton, Qwen3 dense / MoE, Step3.5, Qwen-VL."""
