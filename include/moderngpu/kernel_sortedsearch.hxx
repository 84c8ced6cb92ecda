// Drop-in header name kept for code written against moderngpu 2.x;
// the implementation lives under b200/.
#pragma once
#include "b200/sorted_search.hxx"
