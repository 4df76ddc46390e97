from .helpers import ed_harder_rmse  # noqa: F401
