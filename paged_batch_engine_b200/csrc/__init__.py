from .build import BuildError, build_dir, compile_library, compile_many, load_library

__all__ = ["BuildError", "build_dir", "compile_library", "compile_many", "load_library"]
