#pragma once
#include <cstdio>   // the reference reaches printf through its logging header
