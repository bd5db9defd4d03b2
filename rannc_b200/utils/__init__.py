"""Small helpers (reference: pyrannc/utils.py:1-7)."""


def _to_in_place(p, device):
    p.data = p.to(device)
    return p
