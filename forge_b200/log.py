"""Logging in the reference's manner (src/bindings/logger.cpp, include/forge/logger.h:9-16):

    forge.Logger.set_level(4)                 # 0 none, 1 error, 2 warn, 3 info, 4 debug, 5 trace
    forge.Logger.set_python_sink(callback)    # callback(level, message) instead of stderr; reset_sink() undoes it

At level 4 (debug) the scheduler logs one line per step with its counters (tokens, decodes, prompt portions, requests
waiting and running, free pages per group, preemptions so far); at level 3 (info) the loading of a model and the
compilation of kernel libraries.  The default level is 2.
"""
import sys

NONE, ERROR, WARN, INFO, DEBUG, TRACE = range(6)
_NAMES = {ERROR: "ERROR", WARN: "WARN", INFO: "INFO", DEBUG: "DEBUG", TRACE: "TRACE"}


class Logger:
    _level = WARN
    _sink = None

    @staticmethod
    def set_level(level):
        level = int(level)
        if not NONE <= level <= TRACE:
            raise ValueError(f"log level must be 0..5, got {level}")
        Logger._level = level

    @staticmethod
    def level():
        return Logger._level

    @staticmethod
    def set_python_sink(callback):
        if not callable(callback):
            raise TypeError("the sink must be callable: callback(level, message)")
        Logger._sink = callback

    @staticmethod
    def reset_sink():
        Logger._sink = None

    @staticmethod
    def enabled(level):
        return Logger._level >= level

    @staticmethod
    def log(level, message):
        if Logger._level < level or level == NONE:
            return
        if Logger._sink is not None:
            Logger._sink(level, message)
        else:
            print(f"[forge_b200 {_NAMES[level]}] {message}", file=sys.stderr, flush=True)


def error(msg):
    Logger.log(ERROR, msg)


def warn(msg):
    Logger.log(WARN, msg)


def info(msg):
    Logger.log(INFO, msg)


def debug(msg):
    Logger.log(DEBUG, msg)
