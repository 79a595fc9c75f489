from .flat import SGD, AdamW, LARS

__all__ = ["LARS", "AdamW", "SGD"]
