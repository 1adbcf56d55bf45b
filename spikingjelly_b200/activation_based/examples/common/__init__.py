"""Helpers shared by the reinforcement-learning examples."""
