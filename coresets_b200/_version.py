"""Version of the coresets_b200 package (the sm_100a engine; it tracks its own releases, not the
reference package's)."""
__version__ = "1.0.0.dev0+sm100a"
