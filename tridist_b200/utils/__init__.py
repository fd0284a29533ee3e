from .config import env_flag, env_float, env_int, env_str  # noqa: F401
