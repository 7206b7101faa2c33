"""CompLL front end: lexer, parser and AST for the gradient-compression DSL.

The language is the one the reference generator accepts (functions over
``float*`` / ``uint8*`` vectors with ``lambda_func``, ``reduce``, ``map``,
``range``, ``concat``, ``extract``, ``random<T>``, ``V.size``, sub-byte
``uint<bits>`` vectors; grammar reconstructed from
src/CompLL/GCGen/tree.py:48-660 of mark14wu/hipress), so its two sample sources
parse unchanged, plus what it could not express: float literals (its lexer only
knows digit runs, parser.py:65-72), literal bit widths in ``uint<2>``, comparison
and logical operators as real tokens, the built-in reducers ``smaller`` /
``greater`` / ``sum`` and ``abs`` / ``min`` / ``max`` calls.

Unlike the reference (a token-rewriting translator that copies expression text
through, tree.py:446-507) this front end builds a typed AST with a Pratt
expression parser; the emitter works from the tree.
"""
from __future__ import annotations

import re
from dataclasses import dataclass


class CompileError(Exception):
    def __init__(self, msg, line=None, col=None):
        where = f" at line {line}, column {col}" if line is not None else ""
        super().__init__(msg + where)
        self.line, self.col = line, col


# ------------------------------------------------------------------- lexer
@dataclass
class Token:
    kind: str   # name | int | float | op | eof
    text: str
    line: int
    col: int


_TOKEN_RE = re.compile(r"""
    (?P<ws>\s+) | (?P<comment>//[^\n]*) |
    (?P<float>\d+\.\d*(?:[eE][+-]?\d+)?|\.\d+(?:[eE][+-]?\d+)?|\d+[eE][+-]?\d+) |
    (?P<int>\d+) |
    (?P<name>[A-Za-z_][A-Za-z_0-9]*) |
    (?P<op><<|>>|->|<=|>=|==|!=|&&|\|\||[-+*/%<>=!&|^~(){}\[\],;.?:])
""", re.VERBOSE)


def tokenize(src: str) -> list[Token]:
    out, pos, line, col = [], 0, 1, 1
    while pos < len(src):
        m = _TOKEN_RE.match(src, pos)
        if not m:
            raise CompileError(f"unexpected character {src[pos]!r}", line, col)
        kind = m.lastgroup
        text = m.group()
        if kind not in ("ws", "comment"):
            out.append(Token(kind, text, line, col))
        nl = text.count("\n")
        if nl:
            line += nl
            col = len(text) - text.rfind("\n")
        else:
            col += len(text)
        pos = m.end()
    out.append(Token("eof", "", line, col))
    return out


# --------------------------------------------------------------------- AST
BASIC_BITS = {"uint1": 1, "uint2": 2, "uint4": 4, "uint8": 8, "uint": 32, "int": 32, "float": 32,
              "void": 0, "lambda_func": 0}


@dataclass
class Type:
    name: str                 # basic type name
    bits: "Expr | None" = None  # uint<expr>
    vector: bool = False

    def c_scalar(self) -> str:
        return {"float": "float", "int": "int32_t", "uint": "uint32_t", "uint8": "uint8_t",
                "uint1": "uint8_t", "uint2": "uint8_t", "uint4": "uint8_t", "void": "void"}[self.name]

    def is_subbyte(self) -> bool:
        return self.bits is not None or self.name in ("uint1", "uint2", "uint4")


class Expr:
    pass


@dataclass
class Num(Expr):
    text: str
    is_float: bool


@dataclass
class Name(Expr):
    id: str


@dataclass
class Unary(Expr):
    op: str
    x: Expr


@dataclass
class Binary(Expr):
    op: str
    a: Expr
    b: Expr


@dataclass
class Ternary(Expr):
    c: Expr
    a: Expr
    b: Expr


@dataclass
class Call(Expr):
    fn: str
    args: list


@dataclass
class Index(Expr):
    base: Expr
    idx: Expr


@dataclass
class SizeOf(Expr):
    base: Expr


@dataclass
class Random(Expr):
    type: str
    lo: Expr
    hi: Expr


@dataclass
class Lambda(Expr):
    params: list            # [(Type, name)]
    ret: Type
    body: list              # statements


@dataclass
class Reduce(Expr):
    vec: Expr
    init: Expr
    fn: Expr                # Name of a lambda or built-in reducer


@dataclass
class Map(Expr):
    count: "Expr | None"    # range(count) ...
    vec: "Expr | None"      # ... or a vector to map over
    fn: Expr


@dataclass
class Concat(Expr):
    parts: list


@dataclass
class Extract(Expr):
    src: Expr
    targets: list           # names


# statements
@dataclass
class Decl:
    type: Type
    name: str
    init: "Expr | None"
    line: int = 0


@dataclass
class Assign:
    target: Expr
    value: Expr
    line: int = 0


@dataclass
class If:
    cond: Expr
    then: list
    other: list


@dataclass
class Return:
    value: "Expr | None"


@dataclass
class ExprStmt:
    value: Expr


@dataclass
class Function:
    ret: Type
    name: str
    params: list            # [(Type, name)]
    body: list
    source: str = ""


# ------------------------------------------------------------------ parser
_BINARY_PREC = {"||": 1, "&&": 2, "|": 3, "^": 4, "&": 5, "==": 6, "!=": 6, "<": 7, ">": 7,
                "<=": 7, ">=": 7, "<<": 8, ">>": 8, "+": 9, "-": 9, "*": 10, "/": 10, "%": 10}


class Parser:
    def __init__(self, src: str):
        self.src = src
        self.toks = tokenize(src)
        self.i = 0
        self.no_gt = 0  # >0 while parsing uint<expr>: '>' closes the bracket

    # -- token helpers
    @property
    def tok(self) -> Token:
        return self.toks[self.i]

    def peek(self, k=1) -> Token:
        return self.toks[min(self.i + k, len(self.toks) - 1)]

    def next(self) -> Token:
        t = self.tok
        self.i += 1
        return t

    def accept(self, text) -> bool:
        if self.tok.text == text and self.tok.kind in ("op", "name"):
            self.i += 1
            return True
        return False

    def expect(self, text) -> Token:
        if self.tok.text != text:
            raise CompileError(f"expected {text!r}, found {self.tok.text!r}", self.tok.line, self.tok.col)
        return self.next()

    def expect_name(self) -> str:
        if self.tok.kind != "name":
            raise CompileError(f"expected a name, found {self.tok.text!r}", self.tok.line, self.tok.col)
        return self.next().text

    # -- types
    def at_type(self) -> bool:
        return self.tok.kind == "name" and self.tok.text in BASIC_BITS

    def parse_type(self) -> Type:
        name = self.expect_name()
        if name not in BASIC_BITS:
            raise CompileError(f"cannot resolve typename: {name}", self.tok.line, self.tok.col)
        bits = None
        if name == "uint" and self.tok.text == "<":
            self.next()
            self.no_gt += 1
            bits = self.parse_expr()
            self.no_gt -= 1
            self.expect(">")
        vector = self.accept("*")
        return Type(name, bits, vector)

    # -- program
    def parse_function(self) -> Function:
        # optional leading 'param Name { ... }' blocks are accepted and skipped
        while self.tok.text == "param":
            self.next()
            self.expect_name()
            self.expect("{")
            depth = 1
            while depth:
                t = self.next()
                if t.kind == "eof":
                    raise CompileError("unterminated param block", t.line, t.col)
                depth += t.text == "{"
                depth -= t.text == "}"
        ret = self.parse_type()
        name = self.expect_name()
        self.expect("(")
        params = []
        if not self.accept(")"):
            while True:
                t = self.parse_type()
                params.append((t, self.expect_name()))
                if self.accept(")"):
                    break
                self.expect(",")
        body = self.parse_block()
        return Function(ret, name, params, body, self.src)

    def parse_block(self) -> list:
        self.expect("{")
        out = []
        while not self.accept("}"):
            if self.tok.kind == "eof":
                raise CompileError("missing '}'", self.tok.line, self.tok.col)
            out.append(self.parse_stmt())
        return out

    def parse_body_or_stmt(self) -> list:
        return self.parse_block() if self.tok.text == "{" else [self.parse_stmt()]

    def parse_stmt(self):
        line = self.tok.line
        if self.tok.text == "if":
            self.next()
            self.expect("(")
            cond = self.parse_expr()
            self.expect(")")
            then = self.parse_body_or_stmt()
            other = self.parse_body_or_stmt() if self.accept("else") else []
            return If(cond, then, other)
        if self.tok.text == "return":
            self.next()
            v = None if self.tok.text == ";" else self.parse_expr()
            self.expect(";")
            return Return(v)
        if self.at_type() and (self.peek().kind == "name" or self.peek().text in ("<", "*")):
            ty = self.parse_type()
            name = self.expect_name()
            init = None
            if self.accept("="):
                init = self.parse_rhs()
            self._end_stmt(init)
            return Decl(ty, name, init, line)
        e = self.parse_expr()
        if self.accept("="):
            rhs = self.parse_rhs()
            self._end_stmt(rhs)
            return Assign(e, rhs, line)
        self.expect(";")
        return ExprStmt(e)

    def _end_stmt(self, rhs):
        # the sample sources omit the ';' after a lambda's closing brace
        if isinstance(rhs, Lambda):
            self.accept(";")
        else:
            self.expect(";")

    # -- right-hand sides with special forms
    def parse_rhs(self) -> Expr:
        if self.tok.text == "[" and self.peek().text == "&":
            return self.parse_lambda()
        return self.parse_expr()

    def parse_lambda(self) -> Lambda:
        self.expect("[")
        self.expect("&")
        self.expect("]")
        self.expect("(")
        params = []
        if not self.accept(")"):
            while True:
                t = self.parse_type()
                params.append((t, self.expect_name()))
                if self.accept(")"):
                    break
                self.expect(",")
        self.expect("->")
        ret = self.parse_type()
        return Lambda(params, ret, self.parse_block())

    # -- expressions (precedence climbing)
    def parse_expr(self, min_prec=1) -> Expr:
        lhs = self.parse_unary()
        while True:
            t = self.tok
            if t.kind != "op" or (t.text == ">" and self.no_gt):
                break
            prec = _BINARY_PREC.get(t.text)
            if prec is None or prec < min_prec:
                break
            self.next()
            rhs = self.parse_expr(prec + 1)
            lhs = Binary(t.text, lhs, rhs)
        if min_prec == 1 and self.tok.text == "?":
            self.next()
            a = self.parse_expr()
            self.expect(":")
            b = self.parse_expr()
            lhs = Ternary(lhs, a, b)
        return lhs

    def parse_unary(self) -> Expr:
        if self.tok.kind == "op" and self.tok.text in ("-", "!", "~", "+"):
            op = self.next().text
            return Unary(op, self.parse_unary())
        return self.parse_postfix()

    def parse_postfix(self) -> Expr:
        e = self.parse_primary()
        while True:
            if self.accept("["):
                saved, self.no_gt = self.no_gt, 0
                idx = self.parse_expr()
                self.no_gt = saved
                self.expect("]")
                e = Index(e, idx)
            elif self.tok.text == "." and self.peek().text == "size":
                self.next()
                self.next()
                e = SizeOf(e)
            else:
                return e

    def parse_args(self) -> list:
        args = []
        saved, self.no_gt = self.no_gt, 0
        if not self.accept(")"):
            while True:
                args.append(self.parse_expr())
                if self.accept(")"):
                    break
                self.expect(",")
        self.no_gt = saved
        return args

    def parse_primary(self) -> Expr:
        t = self.tok
        if t.kind == "int":
            self.next()
            return Num(t.text, False)
        if t.kind == "float":
            self.next()
            return Num(t.text, True)
        if t.text == "(":
            self.next()
            saved, self.no_gt = self.no_gt, 0
            e = self.parse_expr()
            self.no_gt = saved
            self.expect(")")
            return e
        if t.kind != "name":
            raise CompileError(f"unrecognized token {t.text!r}", t.line, t.col)
        name = self.next().text
        if name == "random" and self.tok.text == "<":
            self.next()
            ty = self.expect_name()
            self.expect(">")
            self.expect("(")
            a = self.parse_args()
            if len(a) != 2:
                raise CompileError("random<T>(lo, hi) takes two arguments", t.line, t.col)
            return Random(ty, a[0], a[1])
        if self.tok.text != "(":
            return Name(name)
        self.next()
        if name == "reduce":
            a = self.parse_args()
            if len(a) != 3:
                raise CompileError("reduce(vector, init, function) takes three arguments", t.line, t.col)
            return Reduce(a[0], a[1], a[2])
        if name == "map":
            a = self.parse_args()
            if len(a) != 2:
                raise CompileError("map(range(n) | vector, function) takes two arguments", t.line, t.col)
            if isinstance(a[0], Call) and a[0].fn == "range":
                return Map(a[0].args[0], None, a[1])
            return Map(None, a[0], a[1])
        if name == "concat":
            return Concat(self.parse_args())
        if name == "extract":
            a = self.parse_args()
            if len(a) < 2 or not all(isinstance(x, Name) for x in a[1:]):
                raise CompileError("extract(source, name, ...) needs target names", t.line, t.col)
            return Extract(a[0], [x.id for x in a[1:]])
        return Call(name, self.parse_args())


def parse(src: str) -> Function:
    """Parse one DSL function (the unit the generator works on)."""
    p = Parser(src)
    fn = p.parse_function()
    if p.tok.kind != "eof":
        raise CompileError(f"unexpected text after the function: {p.tok.text!r}", p.tok.line, p.tok.col)
    return fn
