def cdiv(a: int, b: int) -> int:
    """Ceiling division (minivllm/utils/utils.py)."""
    return -(-a // b)
