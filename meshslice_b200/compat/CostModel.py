"""Names of CostModel.py mapped to this package."""
from ..cost_model import *  # noqa: F401,F403
