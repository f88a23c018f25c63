"""pytest plugin used when the reference project's own Python test-suite is run against this package.

It does two things the reference's environment would otherwise provide:
  * makes ``import axon`` resolve to ``execution_ucx_b200.axon`` (the reference installs its package
    under the top-level name ``axon``);
  * runs ``async def`` tests (marked ``@pytest.mark.asyncio``) on a fresh event loop, which is what
    pytest-asyncio does in the reference's CI and is not installed here.
"""
import asyncio
import inspect
import sys

import pytest

import execution_ucx_b200.axon as _axon_pkg

sys.modules.setdefault("axon", _axon_pkg)
sys.modules.setdefault("axon.device", _axon_pkg.device)


def pytest_configure(config):
    config.addinivalue_line("markers", "asyncio: run the coroutine test on an event loop")


@pytest.hookimpl(tryfirst=True)
def pytest_pyfunc_call(pyfuncitem):
    fn = pyfuncitem.obj
    if not inspect.iscoroutinefunction(fn):
        return None
    names = pyfuncitem._fixtureinfo.argnames
    kwargs = {n: pyfuncitem.funcargs[n] for n in names}
    loop = asyncio.new_event_loop()
    try:
        asyncio.set_event_loop(loop)
        loop.run_until_complete(asyncio.wait_for(fn(**kwargs), timeout=120))
    finally:
        try:
            loop.run_until_complete(loop.shutdown_asyncgens())
        finally:
            asyncio.set_event_loop(None)
            loop.close()
    return True
