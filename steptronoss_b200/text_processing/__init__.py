"""Text utilities for rewards and evaluation: answer extraction and comparison, repetition scoring,
think/solution splitting."""
