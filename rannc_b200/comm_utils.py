"""Pickled-object broadcast (reference: pyrannc/comm_utils.py:1-8)."""
from .parallel import comm


def bcast_obj(obj, root: int = 0):
    return comm.bcast_obj(obj, root)
