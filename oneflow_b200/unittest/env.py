"""Launch parameters a test run is given through the environment
(reference: python/oneflow/framework/unittest.py:83-128)."""
import os


def eager_execution_enabled():
    return os.getenv("ONEFLOW_TEST_ENABLE_EAGER") == "1"


def typing_check_enabled():
    return os.getenv("ONEFLOW_TEST_ENABLE_TYPING_CHECK") == "1"


def has_node_list():
    return bool(os.getenv("ONEFLOW_TEST_NODE_LIST"))


def node_list():
    s = os.getenv("ONEFLOW_TEST_NODE_LIST")
    if not s:
        raise RuntimeError("ONEFLOW_TEST_NODE_LIST is not set")
    return s.split(",")


def node_size():
    n = os.getenv("ONEFLOW_TEST_NODE_NUM")
    if n:
        return int(n)
    return len(node_list()) if has_node_list() else 1


def has_world_size():
    return True


def world_size():
    from .. import env
    return env.get_world_size()


def device_num():
    s = os.getenv("ONEFLOW_TEST_DEVICE_NUM")
    return int(s) if s else 1
