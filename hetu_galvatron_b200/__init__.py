"""hetu_galvatron_b200: a Blackwell-native automatic hybrid-parallel training system with the
capabilities of Galvatron-2 (profiler, C++ dynamic-programming search engine, hybrid-parallel runtime)."""
__version__ = "0.1.0"
