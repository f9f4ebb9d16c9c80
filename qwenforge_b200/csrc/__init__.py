from .build import KernelLibraryError, build_all, library, library_names, prepare

__all__ = ["KernelLibraryError", "build_all", "library", "library_names", "prepare"]
