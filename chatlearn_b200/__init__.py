"""chatlearn_b200 — a Blackwell-native RL post-training framework."""
__version__ = "0.1.0"
