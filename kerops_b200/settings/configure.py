"""``@configure``: operators whose keyword-only tuning arguments get input-dependent defaults.

Behaviour follows kerops/settings/wrapper.py:12-107 and kerops/settings/utils.py:4-34:

* a parameter annotated ``ConfigurableArg`` must be keyword-only, every keyword-only parameter
  must carry that annotation, and the decorator must name exactly those parameters;
* a configurator is either a constant or a callable whose parameter NAMES select which positional
  arguments of the operator it receives (``lambda x: ...`` gets the operator's ``x``);
* a keyword the caller passes wins over its configurator;
* ``confexc(*excs)`` turns the listed exceptions of a configurator into ``CongiguratorError``;
* ``can_be_configured(**named)`` dry-runs the callable configurators, ``reconfigure`` swaps them.
"""
import functools
import inspect


class ConfigurableArg:
    """Annotation marker for keyword-only, configurable operator arguments."""


class CongiguratorError(Exception):
    """A configurator has no default for these inputs (name spelled as in the reference)."""


_MISSING = object()


def _check_signature(sig, configurator_names):
    confargs = []
    for p in sig.parameters.values():
        is_conf = p.annotation is ConfigurableArg
        is_kwonly = p.kind is inspect.Parameter.KEYWORD_ONLY
        if is_conf and not is_kwonly:
            raise RuntimeError(f'ConfigurableArg must be keyword-only - {p.name}')
        if is_kwonly and not is_conf:
            raise RuntimeError(f'non-ConfigurableArg must not be keyword-only - {p.name}')
        if is_conf:
            confargs.append(p.name)
    _check_match(confargs, configurator_names)
    return confargs


def _check_match(confargs, configurator_names):
    if set(confargs) != set(configurator_names):
        raise RuntimeError(
            f'Configuration mismatch, configurable_args={list(confargs)}, '
            f'configurators_names={list(configurator_names)}'
        )


class ConfiguredFunction:
    def __init__(self, origin_function, **configurators):
        self.origin_function = origin_function
        self.signature = inspect.signature(origin_function)
        self.configurable_args = _check_signature(self.signature, configurators.keys())
        self.usual_args = [
            p.name
            for p in self.signature.parameters.values()
            if p.kind in (inspect.Parameter.POSITIONAL_ONLY, inspect.Parameter.POSITIONAL_OR_KEYWORD)
        ]
        self.configurators = dict(configurators)
        self._make_plans()
        functools.update_wrapper(self, origin_function)

    def _make_plans(self):
        """Per configurable argument: (configurator, positions of the operator arguments it takes) - None for a
        constant, and None as well when a name it asks for is no positional argument of the operator (the call then
        takes the general path and fails there, at call time, as it always did)."""
        self._plans = {}
        for name, conf in self.configurators.items():
            idx = None
            if callable(conf):
                try:
                    idx = tuple(self.usual_args.index(arg) for arg in inspect.signature(conf).parameters)
                except ValueError:
                    idx = None
            self._plans[name] = (conf, idx)
        self._fast = all(idx is not None or not callable(conf) for conf, idx in self._plans.values())

    def _default_for(self, name, positional):
        conf = self.configurators[name]
        if not callable(conf):
            return conf
        wanted = inspect.signature(conf).parameters
        return conf(*(positional[self.usual_args.index(arg)] for arg in wanted))

    def __call__(self, *args, **kwargs):
        # The usual call - every operator argument positional, keywords only for configurable arguments - needs no
        # signature binding: the same result as the general path below at a tenth of its cost.
        if self._fast and len(args) == len(self.usual_args) and all(k in self._plans for k in kwargs):
            final = {}
            for name in self.configurable_args:
                if name in kwargs:
                    final[name] = kwargs[name]
                else:
                    conf, idx = self._plans[name]
                    final[name] = conf if idx is None else conf(*[args[i] for i in idx])
            return self.origin_function(*args, **final)
        filled = {name: kwargs.get(name, _MISSING) for name in self.configurable_args}
        bound = self.signature.bind(*args, **{**kwargs, **filled})
        bound.apply_defaults()
        positional = bound.args
        final = {
            name: (self._default_for(name, positional) if value is _MISSING else value)
            for name, value in bound.kwargs.items()
        }
        return self.origin_function(*positional, **final)

    def can_be_configured(self, **named_args):
        try:
            for conf in self.configurators.values():
                if callable(conf):
                    conf(**{arg: named_args[arg] for arg in inspect.signature(conf).parameters})
        except CongiguratorError:
            return False
        return True

    def reconfigure(self, **new_configurators):
        _check_match(self.configurable_args, new_configurators.keys())
        self.configurators = dict(new_configurators)
        self._make_plans()

    def __repr__(self):
        lines = [f'{self.origin_function.__name__}{self.signature}']
        for name, conf in self.configurators.items():
            if callable(conf):
                shown = 'Configurator(' + ', '.join(inspect.signature(conf).parameters) + ')'
            else:
                shown = str(conf)
            lines.append(f'{name}: {shown}')
        return '\n'.join(lines)


def configure(**configurators):
    def decorate(function):
        return ConfiguredFunction(function, **configurators)

    return decorate


def confexc(*exceptions):
    def decorate(configurator):
        @functools.wraps(configurator)
        def guarded(*args, **kwargs):
            try:
                return configurator(*args, **kwargs)
            except exceptions as e:
                raise CongiguratorError(str(e))

        return guarded

    return decorate
