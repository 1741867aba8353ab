from .awq_marlin import AWQMarlinConfig, AWQMarlinLinearMethod
from .gptq_marlin import GPTQMarlinConfig, GPTQMarlinLinearMethod

__all__ = ["AWQMarlinConfig", "AWQMarlinLinearMethod", "GPTQMarlinConfig", "GPTQMarlinLinearMethod"]
