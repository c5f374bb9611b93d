from .nl import newton_solve

__all__ = ["newton_solve"]
