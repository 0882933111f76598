from . import gaperax, llama, revupel, satavik, tisalorn  # noqa: F401  (register the architectures)
