#pragma once
namespace llis { namespace job { struct InstrumentInfo {}; } }
