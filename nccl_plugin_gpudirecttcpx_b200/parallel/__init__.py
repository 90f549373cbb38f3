from .plugin_env import plugin_env, use_plugin  # noqa: F401
