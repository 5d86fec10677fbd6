"""Rollout flow control between the generation side-car and the RL trainer."""
