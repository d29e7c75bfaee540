"""B200-native drop-in for the `wind_rwkv` package namespace (only `wind_rwkv.rwkv7` exists)."""
__version__ = '0.1'
