"""Shared test helpers: golden fixtures and seeded synthetic inputs."""

import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden(name: str):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def full_rope(half_table: np.ndarray) -> np.ndarray:
    """(S, d/2) -> (S, d): both halves of the head share the rotary angle."""
    return np.concatenate((half_table, half_table), axis=-1)
