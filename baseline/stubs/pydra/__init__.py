"""Stand-in for the `pydra` configuration package, which this image lacks.  Only what the reference's modules
touch at import time and what `ServerConfig()` needs: a base class whose fields are the subclass's class
attributes, `finalize`, and the decorators/aliases its scripts name."""


class Config:
    def __init__(self):
        pass

    def finalize(self):
        pass


def Alias(name):
    return name


def main(config_cls):
    def wrap(fn):
        return fn

    return wrap


def run(fn):
    raise RuntimeError("pydra stand-in: command-line parsing is not provided")


def apply_overrides(config, overrides):
    raise RuntimeError("pydra stand-in: overrides are not provided")
