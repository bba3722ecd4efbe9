"""Typed configurations, one class per architecture, read from ``config.json``."""

from tokenomos_b200.config.darizen import DarizenConfig
from tokenomos_b200.config.fakelorn import FakelornConfig
from tokenomos_b200.config.laposun import LaposunConfig
from tokenomos_b200.config.lfm3 import ConfigError, Lfm3Config, RopeParams

__all__ = ["ConfigError", "DarizenConfig", "FakelornConfig", "LaposunConfig", "Lfm3Config", "RopeParams"]
