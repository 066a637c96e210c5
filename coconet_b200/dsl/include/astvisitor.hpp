// The reference's example programs include <astvisitor.hpp>; in this
// implementation the expression DAG is walked directly and there is nothing
// more to declare.
#pragma once
#include "dsl.hpp"
