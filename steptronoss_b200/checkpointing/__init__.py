"""Native checkpoints (per-rank files + completeness markers + atomic latest pointer) and HF safetensors import/export."""
